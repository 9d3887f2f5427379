"""Sequence-mixing ops over a *packed* token batch: recurrent matrix memories, their short convolutions, latent
attention over a paged cache, group-limited routing, and the fp32-residual norms that surround them.

Packed batch: tokens of all sequences lie one after another along the first axis; ``cu`` (``[R + 1]``) holds the
sequence boundaries, ``slots`` (``[R]``) the row of every sequence in the state tensors.  A sequence may be a whole
prompt, a portion of one, or a single decoded token: what came before lives in the state row (or the paged cache),
which every op reads first and leaves updated.

Every op has a sm_100a kernel (``csrc/seqmix/*.cu`` in ``megatronapp_b200/_C_seq.so``) and a PyTorch fp32 path for
CPU tensors.  CUDA tensors never take the PyTorch path: a missing extension raises.

What is computed in fp32 whatever the activation dtype: the residual stream, norm statistics, decays and gates, the
recurrent state, attention scores and softmax weights, router scores.
"""
from __future__ import annotations

import importlib.util
from collections import Counter
from pathlib import Path
from typing import List, Optional, Sequence, Tuple

import torch
import torch.nn.functional as F

_EXT = None
_EXT_ERR: Optional[BaseException] = None
kernel_calls: Counter = Counter()


def _load_ext():
    global _EXT, _EXT_ERR
    if _EXT is not None or _EXT_ERR is not None:
        return _EXT
    so = Path(__file__).resolve().parent.parent / "_C_seq.so"
    try:
        if not so.exists():
            from ..build import build_seq

            build_seq()
        spec = importlib.util.spec_from_file_location("megatronapp_b200._C_seq", str(so))
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        _EXT = mod
    except BaseException as e:  # noqa: BLE001 - surfaced by ext()
        _EXT_ERR = e
    return _EXT


def ext():
    m = _load_ext()
    if m is None:
        raise RuntimeError(f"megatronapp_b200._C_seq (sm_100a extension) is not available: {_EXT_ERR!r}")
    return m


def have_ext() -> bool:
    return _load_ext() is not None


def _i32(x, device) -> torch.Tensor:
    if torch.is_tensor(x):
        return x.to(device=device, dtype=torch.int32)
    return torch.tensor(list(x), dtype=torch.int32, device=device)


def _host(x) -> List[int]:
    return x.tolist() if torch.is_tensor(x) else list(x)


def _rows3(t: torch.Tensor) -> torch.Tensor:
    """``[T, heads, dim]`` as the kernels take it: contiguous heads, any row stride (a column slice of a fused projection)."""
    return t if (t.stride(2) == 1 and t.stride(1) == t.shape[2]) else t.contiguous()


class PackedBatch:
    """Sequence boundaries and state rows of one packed step, on the host and on the device."""

    def __init__(self, cu: Sequence[int], slots: Sequence[int], device):
        self.cu_host, self.slots_host = _host(cu), _host(slots)
        self.cu = _i32(self.cu_host, device)
        self.slots = _i32(self.slots_host, device)
        self.num_seqs = len(self.slots_host)
        # the sequence of every packed token (the convolution kernel is token-parallel)
        self.tok_seq = _i32([r for r in range(len(self.slots_host)) for _ in range(self.cu_host[r + 1] - self.cu_host[r])], device) \
            if str(device) != "cpu" else None
        self.max_len = max((b - a for a, b in zip(self.cu_host[:-1], self.cu_host[1:])), default=0)

    @classmethod
    def dense(cls, seq_len: int, batch: int, device) -> "PackedBatch":
        """``batch`` independent sequences of ``seq_len`` tokens, stored sequence after sequence."""
        return cls([i * seq_len for i in range(batch + 1)], list(range(batch)), device)


# ---------------------------------------------------------------------------
# norms around an fp32 residual stream
# ---------------------------------------------------------------------------

def add_rms_norm(x: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor, eps: float,
                 out_dtype: torch.dtype, weight_offset: float = 0.0) -> Tuple[torch.Tensor, torch.Tensor]:
    """``x`` fp32 ``[T, h]`` (updated in place by ``+ delta`` when given) -> ``(x, rms_norm(x) * (weight_offset + weight))``;
    the normalised copy leaves in ``out_dtype``, the statistics are fp32.  ``weight_offset = 1`` serves a zero-centred
    weight."""
    if x.is_cuda:
        kernel_calls["add_rms_norm"] += 1
        y = torch.empty(x.shape, dtype=out_dtype, device=x.device)
        ext().add_rms_norm(x, delta if delta is None else delta.contiguous(), weight, y, float(eps), float(weight_offset))
        return x, y
    if delta is not None:
        x.add_(delta.float())
    y = x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * (weight.float() + weight_offset)
    return x, y.to(out_dtype)


def gated_head_rms_norm(o: torch.Tensor, weight: Optional[torch.Tensor], gate: Optional[torch.Tensor], eps: float,
                        out_dtype: torch.dtype, gate_act: str = "sigmoid") -> torch.Tensor:
    """``o`` fp32 ``[T, H, dv]``: every head divided by its own root mean square, times ``weight`` (``[dv]`` shared by
    the heads, or ``[H * dv]``; ``None``: no weight), times ``act(gate)`` (``[T, H * dv]`` pre-activation, any row stride;
    ``gate_act`` is ``"sigmoid"`` or ``"silu"``) -> ``[T, H * dv]``."""
    T, H, dv = o.shape
    if gate_act not in ("sigmoid", "silu"):
        raise ValueError(f"unknown gate activation {gate_act!r}")
    if o.is_cuda:
        kernel_calls["gated_head_rms_norm"] += 1
        y = torch.empty(T, H * dv, dtype=out_dtype, device=o.device)
        ext().gated_head_rms_norm(o.contiguous(), weight, None if gate is None else (gate if gate.stride(1) == 1 else gate.contiguous()),
                                  y, float(eps), gate_act == "silu")
        return y
    y = o * torch.rsqrt(o.pow(2).mean(-1, keepdim=True) + eps)
    if weight is not None:
        w = weight.float()
        y = y * (w.view(1, 1, dv) if w.numel() == dv else w.view(1, H, dv))
    y = y.reshape(T, H * dv)
    if gate is not None:
        y = y * (torch.sigmoid(gate.float()) if gate_act == "sigmoid" else F.silu(gate.float()))
    return y.to(out_dtype)


# ---------------------------------------------------------------------------
# short causal convolution with a carried window
# ---------------------------------------------------------------------------

def causal_conv_silu(x: torch.Tensor, weight: torch.Tensor, pb: PackedBatch, window: torch.Tensor,
                     bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``causal_conv`` followed by SiLU."""
    return causal_conv(x, weight, pb, window, silu=True, bias=bias)


def causal_conv(x: torch.Tensor, weight: torch.Tensor, pb: PackedBatch, window: torch.Tensor, silu: bool = False,
                bias: Optional[torch.Tensor] = None, residual: bool = False) -> torch.Tensor:
    """Depth-wise causal convolution over time, optionally followed by SiLU.  ``x [T, C]``, ``weight [C, taps]`` (last
    column multiplies the current token), ``bias [C]`` (optional), ``window [rows, taps - 1, C]``: the inputs that preceded
    each sequence's first token of this step (zeros at a sequence's start); on return it holds the last ``taps - 1`` inputs
    seen.  ``residual``: the input itself is added to the result (``x + conv(x)``, after the activation if there is one)."""
    if x.is_cuda:
        kernel_calls["causal_conv_silu" if silu else "causal_conv"] += 1
        y = torch.empty(x.shape, dtype=x.dtype, device=x.device)
        ext().causal_conv(x if x.stride(1) == 1 else x.contiguous(), weight.contiguous(), bias, pb.cu, pb.slots, pb.tok_seq,
                          window, y, pb.max_len, bool(silu), bool(residual))
        return y
    taps = weight.shape[1]
    w = weight.float()
    out = []
    for r in range(pb.num_seqs):
        a, b, s = pb.cu_host[r], pb.cu_host[r + 1], pb.slots_host[r]
        if b == a:
            continue
        seq = torch.cat([window[s].float(), x[a:b].float()], dim=0)                # [taps - 1 + n, C]
        y = sum(seq[j:j + (b - a)] * w[:, j] for j in range(taps))
        if bias is not None:
            y = y + bias.float()
        y = F.silu(y) if silu else y
        out.append(y + x[a:b].float() if residual else y)
        if taps > 1:
            window[s] = seq[-(taps - 1):].to(window.dtype)
    return torch.cat(out, dim=0).to(x.dtype)


# ---------------------------------------------------------------------------
# gated delta rule with one decay per key channel
# ---------------------------------------------------------------------------

def delta_rule_scan(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, log_decay: torch.Tensor, beta: torch.Tensor,
                    pb: PackedBatch, state: torch.Tensor, unit_eps: Optional[float] = 1e-6,
                    q_scale: float = 1.0) -> torch.Tensor:
    """``q, k [T, KH, d]``, ``v [T, H, dv]``, ``log_decay [T, H, d]`` (one decay per key channel) or ``[T, H]`` (one per
    head) fp32 (<= 0), ``beta [T, H]`` fp32, ``state [rows, H, d, dv]`` fp32 -> ``o [T, H, dv]`` fp32.  Per head, per token::

        S <- exp(log_decay)[:, None] * S;  u = beta * (v - S^T k);  S <- S + k u^T;  o = S^T q

    Query head ``h`` reads q / k head ``h // (H / KH)``.  With ``unit_eps`` q and k are first scaled to unit length
    (``x / sqrt(sum x^2 + unit_eps)``); q is then multiplied by ``q_scale``."""
    T, H, dv = v.shape
    KH, d = q.shape[1], q.shape[2]
    if q.is_cuda:
        kernel_calls["delta_rule_scan"] += 1
        o = torch.empty(T, H, dv, dtype=torch.float32, device=q.device)
        ext().delta_rule_scan(_rows3(q), _rows3(k), _rows3(v), log_decay.contiguous(), beta.contiguous(),
                              pb.cu, pb.slots, state, o, -1.0 if unit_eps is None else float(unit_eps), float(q_scale),
                              pb.max_len)
        return o
    qf, kf, vf = q.float(), k.float(), v.float()
    if unit_eps is not None:
        qf = qf * torch.rsqrt(qf.pow(2).sum(-1, keepdim=True) + unit_eps)
        kf = kf * torch.rsqrt(kf.pow(2).sum(-1, keepdim=True) + unit_eps)
    qf = qf * q_scale
    rep = H // KH
    if rep > 1:
        qf, kf = qf.repeat_interleave(rep, dim=1), kf.repeat_interleave(rep, dim=1)
    decay = torch.exp(log_decay.float())
    if decay.dim() == 2:
        decay = decay.unsqueeze(-1).expand(T, H, d)
    o = torch.empty(T, H, dv, dtype=torch.float32)
    for r in range(pb.num_seqs):
        a, b, s = pb.cu_host[r], pb.cu_host[r + 1], pb.slots_host[r]
        S = state[s].clone()                                                           # [H, d, dv]
        for t in range(a, b):
            S = S * decay[t].unsqueeze(-1)
            u = beta[t].float().unsqueeze(-1) * (vf[t] - torch.einsum("hdv,hd->hv", S, kf[t]))
            S = S + kf[t].unsqueeze(-1) * u.unsqueeze(1)
            o[t] = torch.einsum("hdv,hd->hv", S, qf[t])
        state[s] = S
    return o


def decay_gates(a_pre: torch.Tensor, b_pre: torch.Tensor, A_log: torch.Tensor, dt_bias: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """The delta rule's gates from the projections' pre-activations ``a_pre [T, C]`` and ``b_pre [T, H]`` (column slices of a
    fused projection are fine), ``A_log [H]``, ``dt_bias [C]`` with ``C = H`` (one decay per head) or ``C = H * d`` (one per key
    channel)::

        log_decay = -exp(A_log[head]) * softplus(a_pre + dt_bias);   beta = sigmoid(b_pre)

    Both fp32, ``[T, C]`` and ``[T, H]``."""
    T, C = a_pre.shape
    H = b_pre.shape[1]
    if a_pre.is_cuda:
        kernel_calls["decay_gates"] += 1
        log_decay = torch.empty(T, C, dtype=torch.float32, device=a_pre.device)
        beta = torch.empty(T, H, dtype=torch.float32, device=a_pre.device)
        ext().decay_gates(a_pre if a_pre.stride(1) == 1 else a_pre.contiguous(), b_pre if b_pre.stride(1) == 1 else b_pre.contiguous(),
                          A_log.contiguous(), dt_bias.contiguous(), log_decay, beta)
        return log_decay, beta
    rate = torch.exp(A_log.float()).repeat_interleave(C // H)
    return -rate * F.softplus(a_pre.float() + dt_bias.float()), torch.sigmoid(b_pre.float())


# ---------------------------------------------------------------------------
# mLSTM matrix memory with stabilised exponential gates
# ---------------------------------------------------------------------------

def mlstm_scan(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, log_i: torch.Tensor, log_f: torch.Tensor,
               pb: PackedBatch, state: torch.Tensor, norm_state: torch.Tensor, max_state: torch.Tensor,
               q_scale: float = 1.0, denom_eps: float = 1e-6) -> torch.Tensor:
    """``q, k [T, H, d]``, ``v [T, H, dv]``, log gates ``log_i, log_f [T, H]`` fp32; ``state [rows, H, d, dv]``,
    ``norm_state [rows, H, d]``, ``max_state [rows, H]`` fp32 (all zero at a sequence's start) -> ``o [T, H, dv]`` fp32::

        m' = max(log_f + m, log_i);  S <- e^(log_f + m - m') S + e^(log_i - m') k v^T;  n likewise with k
        o = S^T q / (max(|n . q|, e^(-m')) + denom_eps)
    """
    T, H, dv = v.shape
    if q.is_cuda:
        kernel_calls["mlstm_scan"] += 1
        o = torch.empty(T, H, dv, dtype=torch.float32, device=q.device)
        ext().mlstm_scan(_rows3(q), _rows3(k), _rows3(v), log_i.contiguous(), log_f.contiguous(),
                         pb.cu, pb.slots, state, norm_state, max_state, o, float(q_scale), float(denom_eps), pb.max_len)
        return o
    qf, kf, vf = q.float() * q_scale, k.float(), v.float()
    li, lf = log_i.float(), log_f.float()
    o = torch.empty(T, H, dv, dtype=torch.float32)
    for r in range(pb.num_seqs):
        a, b, s = pb.cu_host[r], pb.cu_host[r + 1], pb.slots_host[r]
        S, n, m = state[s].clone(), norm_state[s].clone(), max_state[s].clone()
        for t in range(a, b):
            m_new = torch.maximum(lf[t] + m, li[t])
            keep, put = torch.exp(lf[t] + m - m_new), torch.exp(li[t] - m_new)
            S = S * keep.view(H, 1, 1) + put.view(H, 1, 1) * kf[t].unsqueeze(-1) * vf[t].unsqueeze(1)
            n = n * keep.view(H, 1) + put.view(H, 1) * kf[t]
            m = m_new
            den = torch.maximum((n * qf[t]).sum(-1).abs(), torch.exp(-m)) + denom_eps
            o[t] = torch.einsum("hdv,hd->hv", S, qf[t]) / den.unsqueeze(-1)
        state[s], norm_state[s], max_state[s] = S, n, m
    return o


# ---------------------------------------------------------------------------
# latent attention over a paged cache of latents
# ---------------------------------------------------------------------------

def latent_attention_paged(q_lat: torch.Tensor, cache: torch.Tensor, block_table: torch.Tensor, tok_req: torch.Tensor,
                           tok_len: torch.Tensor, block_size: int, scale: float, max_len: int = 0) -> torch.Tensor:
    """Attention of every packed query token over the latents of its own sequence, in the latent space.

    ``q_lat [T, H, r]``: the query of head ``h`` already carried into the latent space (``W_uk,h^T q_h``), so that
    ``score = q_lat . c * scale``; ``cache [num_slots, r]``: one latent per cached token, pages of ``block_size`` slots;
    ``block_table [R, max_blocks]``; ``tok_req [T]`` the sequence of each query token, ``tok_len [T]`` how many cached
    tokens it sees (its own included).  Returns ``sum_j softmax_j(score) c_j`` as fp32 ``[T, H, r]``; the caller applies
    the per-head value up-projection.  Scores, softmax and the weighted sum are fp32.  ``max_len`` (the longest visible
    context, known to the host) lets the kernel split long contexts over several CTAs when the batch has few tokens."""
    T, H, r = q_lat.shape
    if q_lat.is_cuda:
        kernel_calls["latent_attention_paged"] += 1
        o = torch.empty(T, H, r, dtype=torch.float32, device=q_lat.device)
        ext().latent_attention_paged(q_lat.contiguous(), cache, block_table, tok_req, tok_len, o, int(block_size),
                                     float(scale), int(max_len))
        return o
    o = torch.empty(T, H, r, dtype=torch.float32)
    req, lens = tok_req.tolist(), tok_len.tolist()
    t = 0
    while t < T:                                   # tokens of one sequence are contiguous and see growing prefixes
        e = t
        while e + 1 < T and req[e + 1] == req[t]:
            e += 1
        L = lens[e]
        pos = torch.arange(L)
        slots = block_table[req[t]].long()[pos // block_size] * block_size + pos % block_size
        c = cache[slots].float()                                                        # [L, r]
        s = torch.einsum("thr,lr->thl", q_lat[t:e + 1].float(), c) * scale
        vis = pos.view(1, 1, L) < torch.tensor(lens[t:e + 1]).view(-1, 1, 1)
        o[t:e + 1] = torch.einsum("thl,lr->thr", torch.softmax(s.masked_fill(~vis, float("-inf")), -1), c)
        t = e + 1
    return o


# ---------------------------------------------------------------------------
# router: softmax scores, groups ranked by their best expert, top-k inside the kept groups
# ---------------------------------------------------------------------------

def group_limited_router(logits: torch.Tensor, topk: int, num_groups: int, keep_groups: int,
                         renormalize: bool = True) -> Tuple[torch.Tensor, torch.Tensor]:
    """fp32 ``logits [T, E]`` -> dense ``(probs [T, E] fp32, routing_map [T, E] bool)``: softmax over all experts, a
    group of neighbouring experts scores as its best member, only experts of the ``keep_groups`` best groups compete
    for the ``topk`` places; chosen scores are divided by their sum (+ 1e-20) when ``renormalize``."""
    T, E = logits.shape
    if logits.is_cuda:
        kernel_calls["group_limited_router"] += 1
        probs = torch.zeros(T, E, dtype=torch.float32, device=logits.device)
        rmap = torch.zeros(T, E, dtype=torch.bool, device=logits.device)
        ext().group_limited_router(logits.float().contiguous(), probs, rmap, int(topk), int(num_groups), int(keep_groups),
                                   bool(renormalize))
        return probs, rmap
    s = torch.softmax(logits.float(), dim=-1)
    best = s.view(T, num_groups, E // num_groups).amax(-1)
    kept = torch.zeros(T, num_groups, dtype=torch.bool).scatter_(1, torch.topk(best, keep_groups, dim=-1).indices, True)
    masked = s.masked_fill(~kept.repeat_interleave(E // num_groups, dim=1), -1.0)
    idx = torch.topk(masked, topk, dim=-1).indices
    w = torch.gather(s, 1, idx)
    if renormalize:
        w = w / (w.sum(-1, keepdim=True) + 1e-20)
    return torch.zeros_like(s).scatter_(1, idx, w), torch.zeros(T, E, dtype=torch.bool).scatter_(1, idx, True)


# ---------------------------------------------------------------------------
# norm on a sublayer's output, fused with the fp32 residual addition
# ---------------------------------------------------------------------------

def _rms(t: torch.Tensor, eps: float) -> torch.Tensor:
    return t * torch.rsqrt(t.pow(2).mean(-1, keepdim=True) + eps)


def norm_add(x: torch.Tensor, a: torch.Tensor, weight: Optional[torch.Tensor], eps: float, out_dtype: torch.dtype,
             weight_offset: float = 0.0, b: Optional[torch.Tensor] = None, weight_a: Optional[torch.Tensor] = None,
             weight_b: Optional[torch.Tensor] = None, extra: Optional[torch.Tensor] = None,
             next_weight: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """``x`` fp32 ``[T, h]`` is updated in place by ``+ rms_norm(m) * (weight_offset + weight) + extra`` and returned with
    a second tensor in ``out_dtype``.  ``m`` is the sublayer output ``a``; with a second branch ``b`` it is the mean of the two
    branches, each RMS-normed with its own plain weight: ``(rms_norm(a) * weight_a + rms_norm(b) * weight_b) / 2``.
    ``weight = None``: ``m`` is added as it is, without the outer norm.  ``extra`` (optional) is another sublayer's output added
    in the same pass.  The second tensor is the new ``x`` itself, or with ``next_weight`` its RMS norm times that weight (the
    input of the sublayer that follows)."""
    if x.is_cuda:
        kernel_calls["norm_add"] += 1
        y = torch.empty(x.shape, dtype=out_dtype, device=x.device)
        ext().norm_add(x, a.contiguous(), None if b is None else b.contiguous(), weight_a, weight_b, weight, y, float(eps),
                       float(weight_offset), None if extra is None else extra.contiguous(), next_weight)
        return x, y
    m = a.float()
    if b is not None:
        m = 0.5 * (_rms(m, eps) * weight_a.float() + _rms(b.float(), eps) * weight_b.float())
    if weight is not None:
        m = _rms(m, eps) * (weight.float() + weight_offset)
    if extra is not None:
        m = m + extra.float()
    x.add_(m)
    y = x if next_weight is None else _rms(x, eps) * next_weight.float()
    return x, y.to(out_dtype)


# ---------------------------------------------------------------------------
# whole-projection q / k norm + partial interleaved rotary positions
# ---------------------------------------------------------------------------

def norm_rope(q: torch.Tensor, k: torch.Tensor, weight_q: torch.Tensor, weight_k: torch.Tensor, positions: torch.Tensor,
              inv_freq: torch.Tensor, head_dim: int, rot_dims: int, eps: float) -> Tuple[torch.Tensor, torch.Tensor]:
    """``q [T, H * d]`` and ``k [T, G * d]`` (column slices of a fused projection are fine): each is RMS-normed over its
    whole row with a weight per channel, then the first ``rot_dims`` dimensions of every head are rotated, dimension
    ``2i`` paired with ``2i + 1``, by the angle ``positions[t] * inv_freq[i]`` (fp32).  Returns contiguous ``(q, k)``."""
    if q.is_cuda:
        kernel_calls["norm_rope"] += 1
        qo = torch.empty(q.shape, dtype=q.dtype, device=q.device)
        ko = torch.empty(k.shape, dtype=k.dtype, device=k.device)
        ext().norm_rope(q if q.stride(1) == 1 else q.contiguous(), k if k.stride(1) == 1 else k.contiguous(), weight_q, weight_k,
                        positions.contiguous(), inv_freq, qo, ko, int(head_dim), int(rot_dims), float(eps))
        return qo, ko
    ang = positions.float().unsqueeze(-1) * inv_freq.float()                          # [T, rot / 2]
    cs, sn = torch.cos(ang).unsqueeze(1), torch.sin(ang).unsqueeze(1)
    outs = []
    for t, w in ((q, weight_q), (k, weight_k)):
        y = (_rms(t.float(), eps) * w.float()).view(t.shape[0], -1, head_dim).clone()
        u, v = y[..., 0:rot_dims:2].clone(), y[..., 1:rot_dims:2].clone()
        y[..., 0:rot_dims:2] = u * cs - v * sn
        y[..., 1:rot_dims:2] = v * cs + u * sn
        outs.append(y.view(t.shape).to(t.dtype))
    return outs[0], outs[1]


# ---------------------------------------------------------------------------
# paged grouped-query attention whose softmax weights are mixed across heads
# ---------------------------------------------------------------------------

def mixed_attention_paged(q: torch.Tensor, kcache: torch.Tensor, vcache: torch.Tensor, block_table: torch.Tensor,
                          tok_req: torch.Tensor, tok_len: torch.Tensor, block_size: int, scale: float,
                          talk: Optional[torch.Tensor] = None, gate: Optional[torch.Tensor] = None, max_len: int = 0,
                          force_generic: bool = False) -> torch.Tensor:
    """``q [T, H, d]`` against paged keys ``[slots, G, d]`` and values ``[slots, G, dv]``: per head the ordinary softmax
    over the ``tok_len[t]`` visible keys of the token's sequence; the weights of all heads are then mixed,
    ``M_h = sum_g talk[h, g] P_g`` (``talk`` fp32 ``[H, H]``; ``None``: no mixing), and head ``h`` applies ``M_h`` to the
    values of its own key/value head ``h // (H / G)``.  ``gate [T, H * dv]`` (pre-activation) multiplies the result by
    its sigmoid.  Scores, weights and sums are fp32.  Returns ``[T, H * dv]`` in ``q``'s dtype.  Head sizes that 16-byte
    vectors divide take the vector kernel (several queries of a prompt per CTA), others the scalar one (``force_generic``
    selects it regardless, for tests)."""
    T, H, d = q.shape
    G, dv = kcache.shape[1], vcache.shape[2]
    if q.is_cuda:
        kernel_calls["mixed_attention_paged"] += 1
        o = torch.empty(T, H * dv, dtype=q.dtype, device=q.device)
        ext().mixed_attention_paged(_rows3(q), kcache, vcache, block_table, tok_req, tok_len,
                                    None if talk is None else talk.float().contiguous(),
                                    None if gate is None else (gate if gate.stride(1) == 1 else gate.contiguous()), o,
                                    int(block_size), float(scale), int(max_len), bool(force_generic))
        return o
    o = torch.empty(T, H, dv, dtype=torch.float32)
    req, lens = tok_req.tolist(), tok_len.tolist()
    rep = H // G
    t = 0
    while t < T:
        e = t
        while e + 1 < T and req[e + 1] == req[t]:
            e += 1
        L = max(lens[t:e + 1])
        pos = torch.arange(L)
        slots = block_table[req[t]].long()[pos // block_size] * block_size + pos % block_size
        kk = kcache[slots].float().repeat_interleave(rep, dim=1)                        # [L, H, d]
        vv = vcache[slots].float().repeat_interleave(rep, dim=1)
        s = torch.einsum("thd,lhd->htl", q[t:e + 1].float(), kk) * scale
        vis = pos.view(1, 1, L) < torch.tensor(lens[t:e + 1]).view(1, -1, 1)
        P = torch.softmax(s.masked_fill(~vis, float("-inf")), -1)
        if talk is not None:
            P = torch.einsum("hg,gtl->htl", talk.float(), P)
        o[t:e + 1] = torch.einsum("htl,lhv->thv", P, vv)
        t = e + 1
    o = o.reshape(T, H * dv)
    if gate is not None:
        o = o * torch.sigmoid(gate.float())
    return o.to(q.dtype)


# ---------------------------------------------------------------------------
# generalized delta rule: per-channel decay and removal along the unit key
# ---------------------------------------------------------------------------

def gen_delta_scan(r: torch.Tensor, k: torch.Tensor, v: torch.Tensor, w_pre: torch.Tensor, a_pre: torch.Tensor,
                   w_bias: Optional[torch.Tensor], pb: PackedBatch, state: torch.Tensor, decay_scale: float,
                   unit_eps: float = 1e-6) -> torch.Tensor:
    """``r, k [T, H, d]``, ``v [T, H, dv]``, pre-activations ``w_pre, a_pre [T, H * d]``, ``state [rows, H, d, dv]`` fp32
    -> ``o [T, H, dv]`` fp32.  Per head and token, with ``u = k / sqrt(sum k^2 + unit_eps)``::

        w = exp(-decay_scale * sigmoid(w_pre + w_bias));  a = sigmoid(a_pre)
        S <- diag(w) S - (a * u) (u^T S) + k v^T   (decay and removal both act on the previous S);   o = S^T r
    """
    T, H, dv = v.shape
    d = r.shape[2]
    if r.is_cuda:
        kernel_calls["gen_delta_scan"] += 1
        o = torch.empty(T, H, dv, dtype=torch.float32, device=r.device)
        ext().gen_delta_scan(_rows3(r), _rows3(k), _rows3(v), w_pre if w_pre.stride(1) == 1 else w_pre.contiguous(),
                             a_pre if a_pre.stride(1) == 1 else a_pre.contiguous(), w_bias, pb.cu, pb.slots, state, o,
                             float(decay_scale), float(unit_eps), pb.max_len)
        return o
    rf, kf, vf = r.float(), k.float(), v.float()
    wz = w_pre.float() + (w_bias.float() if w_bias is not None else 0.0)
    w = torch.exp(-decay_scale * torch.sigmoid(wz)).view(T, H, d)
    a = torch.sigmoid(a_pre.float()).view(T, H, d)
    u = kf * torch.rsqrt(kf.pow(2).sum(-1, keepdim=True) + unit_eps)
    au = a * u
    o = torch.empty(T, H, dv, dtype=torch.float32)
    for s_ in range(pb.num_seqs):
        lo, hi, row = pb.cu_host[s_], pb.cu_host[s_ + 1], pb.slots_host[s_]
        S = state[row].clone()
        for t in range(lo, hi):
            proj = torch.einsum("hd,hdv->hv", u[t], S)
            S = w[t].unsqueeze(-1) * S - au[t].unsqueeze(-1) * proj.unsqueeze(1) + kf[t].unsqueeze(-1) * vf[t].unsqueeze(1)
            o[t] = torch.einsum("hdv,hd->hv", S, rf[t])
        state[row] = S
    return o


# ---------------------------------------------------------------------------
# minGRU
# ---------------------------------------------------------------------------

def mingru_scan(z_pre: torch.Tensor, u_pre: torch.Tensor, g_pre: torch.Tensor, pb: PackedBatch, state: torch.Tensor) -> torch.Tensor:
    """Pre-activations ``z_pre, u_pre, g_pre [T, C]``, ``state [rows, C]`` fp32 -> ``[T, C]`` in the inputs' dtype::

        z = sigmoid(z_pre);  c = u_pre + 1/2 where u_pre >= 0, sigmoid(u_pre) elsewhere
        S <- (1 - z) S + z c;  y = S * silu(g_pre)
    """
    if z_pre.is_cuda:
        kernel_calls["mingru_scan"] += 1
        y = torch.empty(z_pre.shape, dtype=z_pre.dtype, device=z_pre.device)
        fix = lambda t: t if t.stride(1) == 1 else t.contiguous()  # noqa: E731
        ext().mingru_scan(fix(z_pre), fix(u_pre), fix(g_pre), pb.cu, pb.slots, state, y, pb.max_len)
        return y
    z, u = torch.sigmoid(z_pre.float()), u_pre.float()
    cand = torch.where(u >= 0, u + 0.5, torch.sigmoid(u))
    out = torch.empty(z.shape, dtype=torch.float32)
    for s_ in range(pb.num_seqs):
        lo, hi, row = pb.cu_host[s_], pb.cu_host[s_ + 1], pb.slots_host[s_]
        S = state[row].clone()
        for t in range(lo, hi):
            S = (1 - z[t]) * S + z[t] * cand[t]
            out[t] = S
        state[row] = S
    return (out * F.silu(g_pre.float())).to(z_pre.dtype)


# ---------------------------------------------------------------------------
# clamped gated activation
# ---------------------------------------------------------------------------

def clamped_glu(x: torch.Tensor, limit: float, alpha: float = 1.702, shift: float = 1.0) -> torch.Tensor:
    """``x [..., 2 F]`` holding ``[gate | up]`` -> ``[..., F]``: ``g = min(gate, limit)``, ``u = clamp(up, -limit, limit)``,
    ``y = g * sigmoid(alpha * g) * (u + shift)``."""
    F_ = x.shape[-1] // 2
    if x.is_cuda:
        kernel_calls["clamped_glu"] += 1
        x2 = x.reshape(-1, x.shape[-1])
        y = torch.empty(x2.shape[0], F_, dtype=x.dtype, device=x.device)
        ext().clamped_glu(x2 if x2.stride(1) == 1 else x2.contiguous(), y, float(limit), float(alpha), float(shift))
        return y.view(*x.shape[:-1], F_)
    g = torch.clamp(x[..., :F_].float(), max=limit)
    u = torch.clamp(x[..., F_:].float(), -limit, limit)
    return (g * torch.sigmoid(alpha * g) * (u + shift)).to(x.dtype)


# ---------------------------------------------------------------------------
# several fp32 residual streams: update by a sublayer's output fused with the norm of the next sublayer's input
# ---------------------------------------------------------------------------

def stream_mix_norm(x: torch.Tensor, a: Optional[torch.Tensor] = None, b: Optional[torch.Tensor] = None,
                    bias_a: Optional[torch.Tensor] = None, ls: Optional[torch.Tensor] = None, scale_a: float = 1.0,
                    scale_b: float = 1.0, mix: Optional[torch.Tensor] = None, outc: Optional[torch.Tensor] = None,
                    inp: Optional[torch.Tensor] = None, weight: Optional[torch.Tensor] = None, beta: Optional[torch.Tensor] = None,
                    eps: float = 1e-5, out_dtype: Optional[torch.dtype] = None, center: bool = True):
    """``x`` fp32 ``[T, S, W]``: ``S`` residual streams, updated in place.  With a pending sublayer output ``a [T, W]``
    (and optionally a second branch ``b``)::

        y = ls * (scale_a * (a + bias_a) + scale_b * b);   x_t <- sum_s mix[s, t] x_s + outc[t] * y   (all t at once)

    then, with read weights ``inp [S]``: ``u = sum_s inp[s] x_s`` and ``h = norm(u) * weight + beta`` (layer norm when
    ``center``, else RMS norm), in ``out_dtype``.  ``mix``, ``outc``, ``inp`` are fp32; everything is computed in fp32.
    Returns ``(x, h or None)``."""
    T, S, W = x.shape
    if x.is_cuda:
        kernel_calls["stream_mix_norm"] += 1
        h = torch.empty(T, W, dtype=out_dtype or weight.dtype, device=x.device) if inp is not None else None
        fix = lambda t: t if (t is None or t.stride(1) == 1) else t.contiguous()  # noqa: E731
        ext().stream_mix_norm(x, fix(a), fix(b), bias_a, ls, float(scale_a), float(scale_b), mix, outc, inp, weight, beta, h,
                              float(eps), bool(center))
        return x, h
    if a is not None:
        y = a.float()
        if bias_a is not None:
            y = y + bias_a.float()
        y = y * scale_a
        if b is not None:
            y = y + scale_b * b.float()
        if ls is not None:
            y = y * ls.float()
        x.copy_(torch.einsum("st,nsw->ntw", mix.float(), x) + outc.float().view(1, S, 1) * y.unsqueeze(1))
    if inp is None:
        return x, None
    u = torch.einsum("s,nsw->nw", inp.float(), x)
    if center:
        u = u - u.mean(-1, keepdim=True)
    h = u * torch.rsqrt(u.pow(2).mean(-1, keepdim=True) + eps) * weight.float()
    if beta is not None:
        h = h + beta.float()
    return x, h.to(out_dtype or weight.dtype)


def add_sinusoid(x: torch.Tensor, positions: torch.Tensor, freq: torch.Tensor) -> torch.Tensor:
    """``x`` fp32 ``[T, W]`` (in place): entry ``2i`` gains ``sin(positions[t] * freq[i])``, entry ``2i + 1`` the cosine;
    ``freq`` fp32 ``[W / 2]``.  Angles are fp32."""
    if x.is_cuda:
        kernel_calls["add_sinusoid"] += 1
        ext().add_sinusoid(x, positions.contiguous().long(), freq)
        return x
    ang = positions.float().unsqueeze(-1) * freq.float()
    x[:, 0::2] += torch.sin(ang)
    x[:, 1::2] += torch.cos(ang)
    return x


def head_rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """``x [T, heads, d]`` (a column slice of a fused projection is fine): every head divided by its root mean square over
    ``d`` (fp32 statistics), times ``weight [d]`` shared by the heads.  Returns a contiguous tensor in ``x``'s dtype."""
    if x.is_cuda:
        kernel_calls["head_rms_norm"] += 1
        y = torch.empty(x.shape, dtype=x.dtype, device=x.device)
        ext().head_rms_norm(_rows3(x), weight, y, float(eps))
        return y
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * weight.float()).to(x.dtype)


# ---------------------------------------------------------------------------
# paged grouped-query attention: sliding window, distance penalty per head, sink in the denominator, gate per head
# ---------------------------------------------------------------------------

def window_attention_paged(q: torch.Tensor, kcache: torch.Tensor, vcache: torch.Tensor, block_table: torch.Tensor,
                           tok_req: torch.Tensor, tok_len: torch.Tensor, block_size: int, scale: float, window: int = 0,
                           slopes: Optional[torch.Tensor] = None, sink: bool = False, gate: Optional[torch.Tensor] = None,
                           out_scale: float = 1.0, max_len: int = 0, dist_bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``q [T, H, d]`` against paged keys ``[slots, G, d]`` and values ``[slots, G, dv]``.  The token at position
    ``i = tok_len[t] - 1`` sees the keys ``j`` of its own sequence with ``0 <= i - j < window`` (``window = 0``: all up to
    ``i``)::

        s_j = q . k_j * scale - slopes[h] * (i - j) + dist_bias[min(i - j, L - 1), h];   p_j = exp(s_j) / (sink + sum_j exp(s_j))

    ``dist_bias`` (optional) is an fp32 table ``[L, H]`` of additive biases by distance; distances beyond its last row use the
    last row.

    ``sink``: a key of score 0 without a value takes part in the normalisation.  ``gate [T, H]`` (pre-activation) multiplies
    head ``h``'s output by its sigmoid; ``out_scale`` multiplies everything.  Scores, weights and sums are fp32.  Returns
    ``[T, H * dv]`` in ``q``'s dtype.  ``max_len`` (the longest context, known to the host) lets a batch with one token per
    sequence (``block_table`` has as many rows as ``q``) split its keys over several CTAs."""
    T, H, d = q.shape
    G, dv = kcache.shape[1], vcache.shape[2]
    if q.is_cuda:
        kernel_calls["window_attention_paged"] += 1
        o = torch.empty(T, H * dv, dtype=q.dtype, device=q.device)
        ext().window_attention_paged(_rows3(q), kcache, vcache, block_table, tok_req, tok_len,
                                     None if slopes is None else slopes.float().contiguous(),
                                     None if gate is None else (gate if gate.stride(1) == 1 else gate.contiguous()), o,
                                     int(block_size), float(scale), int(window), bool(sink), float(out_scale), int(max_len),
                                     None if dist_bias is None else dist_bias.float().contiguous())
        return o
    o = torch.empty(T, H, dv, dtype=torch.float32)
    req, lens = tok_req.tolist(), tok_len.tolist()
    rep = H // G
    t = 0
    while t < T:
        e = t
        while e + 1 < T and req[e + 1] == req[t]:
            e += 1
        L = max(lens[t:e + 1])
        lo = max(0, min(lens[t:e + 1]) - window) if window > 0 else 0
        pos = torch.arange(lo, L)
        slots = block_table[req[t]].long()[pos // block_size] * block_size + pos % block_size
        kk = kcache[slots].float().repeat_interleave(rep, dim=1)                        # [L - lo, H, d]
        vv = vcache[slots].float().repeat_interleave(rep, dim=1)
        s = torch.einsum("thd,lhd->htl", q[t:e + 1].float(), kk) * scale
        qpos = torch.tensor(lens[t:e + 1]).view(1, -1, 1) - 1
        dist = qpos - pos.view(1, 1, -1)
        if slopes is not None:
            s = s - slopes.float().view(H, 1, 1) * dist
        if dist_bias is not None:
            idx = dist[0].clamp(0, dist_bias.shape[0] - 1)                              # [n, L]
            s = s + dist_bias.float()[idx].permute(2, 0, 1)
        vis = (dist >= 0) & ((dist < window) if window > 0 else torch.ones_like(dist, dtype=torch.bool))
        s = s.masked_fill(~vis, float("-inf"))
        m = s.amax(-1, keepdim=True)
        m = torch.clamp(m, min=0.0) if sink else torch.where(torch.isinf(m), torch.zeros_like(m), m)
        ex = torch.exp(s - m)
        den = ex.sum(-1, keepdim=True) + (torch.exp(-m) if sink else 0.0)
        P = ex / torch.where(den > 0, den, torch.ones_like(den))
        o[t:e + 1] = torch.einsum("htl,lhv->thv", P, vv)
        t = e + 1
    if gate is not None:
        o = o * torch.sigmoid(gate.float()).unsqueeze(-1)
    return (o * out_scale).reshape(T, H * dv).to(q.dtype)


# ---------------------------------------------------------------------------
# selective scan: one decay per channel and state, step size per channel
# ---------------------------------------------------------------------------

def selective_scan(x: torch.Tensor, dt_pre: torch.Tensor, B: torch.Tensor, C: torch.Tensor, A_log: torch.Tensor, D: torch.Tensor,
                   pb: PackedBatch, state: torch.Tensor, z: Optional[torch.Tensor] = None, dt_bias: Optional[torch.Tensor] = None,
                   out_scale: float = 1.0) -> torch.Tensor:
    """``x [T, C]``, step sizes before bias and softplus ``dt_pre [T, C]`` fp32, ``B, C [T, N]``, ``A_log [C, N]``, ``D [C]``,
    ``state [rows, C, N]`` fp32 -> ``[T, C]`` in ``x``'s dtype.  Per channel ``c`` and state ``n``::

        dt = softplus(dt_pre + dt_bias);   S[c, n] <- exp(-dt_c exp(A_log[c, n])) S[c, n] + dt_c x_c B_n
        y_c = sum_n S[c, n] C_n + D_c x_c;   y <- y * silu(z) * out_scale

    Step sizes, decays and the state are fp32."""
    T, Cn = x.shape
    N = B.shape[1]
    if x.is_cuda:
        kernel_calls["selective_scan"] += 1
        y = torch.empty(T, Cn, dtype=x.dtype, device=x.device)
        fix = lambda t: t if (t is None or t.stride(1) == 1) else t.contiguous()  # noqa: E731
        ext().selective_scan(fix(x), fix(z), fix(B), fix(C), fix(dt_pre.float()), dt_bias, A_log.contiguous(), D, pb.cu, pb.slots,
                             state, y, float(out_scale))
        return y
    xf, Bf, Cf = x.float(), B.float(), C.float()
    dt = F.softplus(dt_pre.float() + (dt_bias.float() if dt_bias is not None else 0.0), threshold=20.0)
    A = -torch.exp(A_log.float())
    out = torch.empty(T, Cn, dtype=torch.float32)
    for r in range(pb.num_seqs):
        lo, hi, row = pb.cu_host[r], pb.cu_host[r + 1], pb.slots_host[r]
        S = state[row].clone()
        for t in range(lo, hi):
            S = torch.exp(dt[t].unsqueeze(-1) * A) * S + (dt[t] * xf[t]).unsqueeze(-1) * Bf[t].unsqueeze(0)
            out[t] = S @ Cf[t] + D.float() * xf[t]
        state[row] = S
    if z is not None:
        out = out * F.silu(z.float())
    return (out * out_scale).to(x.dtype)


# ---------------------------------------------------------------------------
# retention: matrix memory with a fixed decay per head, no normaliser; rotary positions applied on the way in
# ---------------------------------------------------------------------------

def rotary_frequencies(rot_dims: int, base: float, device=None) -> Optional[torch.Tensor]:
    """``base^(-2 i / rot_dims)`` for ``i = 0 .. rot_dims / 2 - 1`` (computed in fp64, returned as fp32); ``None`` when nothing rotates."""
    if rot_dims <= 0:
        return None
    i = torch.arange(rot_dims // 2, dtype=torch.float64)
    return torch.pow(torch.tensor(float(base), dtype=torch.float64), -2.0 * i / rot_dims).float().to(device)


def retention_scan(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, decay: torch.Tensor, pb: PackedBatch, state: torch.Tensor,
                   positions: Optional[torch.Tensor] = None, inv_freq: Optional[torch.Tensor] = None, k_scale: float = 1.0) -> torch.Tensor:
    """``q, k [T, H, d]``, ``v [T, H, dv]``, ``decay [H]`` fp32, ``state [rows, H, d, dv]`` fp32 -> ``o [T, H, dv]`` fp32::

        S <- decay_h * S + (k_scale * k) v^T;   o = S^T q

    With ``inv_freq [n]`` (fp32) the first ``2 n`` dimensions of every q and k head are rotated first, dimension ``i`` paired
    with ``i + n`` by the angle ``positions[t] * inv_freq[i]``: ``(u, w) -> (u cos - w sin, w cos + u sin)``.  Angles,
    rotated vectors and the state are fp32."""
    T, H, dv = v.shape
    d = q.shape[2]
    n_rot = 0 if inv_freq is None else int(inv_freq.numel())
    if n_rot and positions is None:
        raise ValueError("retention_scan: rotation needs positions")
    if q.is_cuda:
        kernel_calls["retention_scan"] += 1
        o = torch.empty(T, H, dv, dtype=torch.float32, device=q.device)
        ext().retention_scan(_rows3(q), _rows3(k), _rows3(v), decay.float().contiguous(),
                             None if not n_rot else positions.contiguous().long(), None if not n_rot else inv_freq.float().contiguous(),
                             pb.cu, pb.slots, state, o, float(k_scale), pb.max_len)
        return o
    qf, kf, vf = q.float().clone(), k.float().clone(), v.float()
    if n_rot:
        ang = positions.float().unsqueeze(-1) * inv_freq.float()                       # [T, n]
        cs, sn = torch.cos(ang).unsqueeze(1), torch.sin(ang).unsqueeze(1)
        for t in (qf, kf):
            u, w = t[..., :n_rot].clone(), t[..., n_rot:2 * n_rot].clone()
            t[..., :n_rot] = u * cs - w * sn
            t[..., n_rot:2 * n_rot] = w * cs + u * sn
    kf = kf * k_scale
    dec = decay.float().view(H, 1, 1)
    o = torch.empty(T, H, dv, dtype=torch.float32)
    for r in range(pb.num_seqs):
        a, b, s = pb.cu_host[r], pb.cu_host[r + 1], pb.slots_host[r]
        S = state[s].clone()
        for t in range(a, b):
            S = dec * S + kf[t].unsqueeze(-1) * vf[t].unsqueeze(1)
            o[t] = torch.einsum("hdv,hd->hv", S, qf[t])
        state[s] = S
    return o


# ---------------------------------------------------------------------------
# polynomial activation of normalised powers
# ---------------------------------------------------------------------------

def poly_norm(z: torch.Tensor, coef: torch.Tensor, eps: float) -> torch.Tensor:
    """``z [..., F]``, ``coef [4] = (a, b, c, e)``: ``a N(z) + b N(z^2) + c N(z^3) + e`` with element-wise powers and ``N`` the
    division of a row by its root mean square (``eps`` inside the root).  Statistics and the sum are fp32; the result
    leaves in ``z``'s dtype."""
    F_ = z.shape[-1]
    if z.is_cuda:
        kernel_calls["poly_norm"] += 1
        z2 = z.reshape(-1, F_)
        y = torch.empty(z2.shape[0], F_, dtype=z.dtype, device=z.device)
        ext().poly_norm(z2 if z2.stride(1) == 1 else z2.contiguous(), coef.float().contiguous(), y, float(eps))
        return y.view(z.shape)
    zf, c = z.float(), coef.float()
    return (c[0] * _rms(zf, eps) + c[1] * _rms(zf * zf, eps) + c[2] * _rms(zf * zf * zf, eps) + c[3]).to(z.dtype)


# ---------------------------------------------------------------------------
# tanh-GELU gate times a per-token vector
# ---------------------------------------------------------------------------

def gelu_mul(g: torch.Tensor, e: torch.Tensor) -> torch.Tensor:
    """``gelu_tanh(g) * e`` for ``g, e [T, n]`` (``e`` may be a column slice of a wider table), computed in fp32, in ``g``'s dtype;
    ``gelu_tanh(z) = z / 2 * (1 + tanh(sqrt(2 / pi) * (z + 0.044715 z^3)))``."""
    if g.is_cuda:
        kernel_calls["gelu_mul"] += 1
        y = torch.empty(g.shape, dtype=g.dtype, device=g.device)
        ext().gelu_mul(g if g.stride(1) == 1 else g.contiguous(), e if e.stride(1) == 1 else e.contiguous(), y)
        return y
    return (F.gelu(g.float(), approximate="tanh") * e.float()).to(g.dtype)
