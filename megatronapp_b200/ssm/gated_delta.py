"""Gated delta-rule mixer with one decay per head and key channel, or one per head.

Per head a matrix memory ``S [d, dv]`` is carried from token to token::

    g = exp(-exp(A_log) * softplus(W_a2 W_a1 h + dt_bias))          (one value per key channel)
    S <- g[:, None] * S;  u = beta * (v - S^T k);  S <- S + k u^T;  o = S^T q

with ``beta = sigmoid(W_b h)``.  q, k and v come out of a short causal depth-wise convolution + SiLU; q and k are then
normalised to unit length head by head (q additionally times ``d^-1/2``).  The read-out is RMS-normalised per head with
one weight vector common to all heads and gated by ``sigmoid(W_g2 W_g1 h)``.  Grouped heads: value head ``h`` uses q / k head
``h // (heads / kv_heads)``.

Variants, all parameters: ``decay_per_head`` (``g`` is one value per head: ``W_a`` has ``heads`` rows and ``dt_bias`` ``heads``
entries); ``decay_rank = 0`` / ``gate_rank = 0`` (the decay's / the gate's pre-activation comes straight out of the input
projection, without the low-rank pair); ``gate_act = "silu"`` (the read-out is multiplied by ``silu`` of the gate instead of its
sigmoid).

The module keeps the framework's Mamba mixer shape (``ssm/mamba.py``): one fused input projection whose rows are the
segments ``[q | k | v | a1 | g1 | b]``, one convolution over the ``[q | k | v]`` channels, state in the inference
context (convolution window + fp32 memory per sequence), row-parallel output projection.  Decays, gates, unit norms and
the state are fp32 whatever the parameter dtype.
"""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..ops import seqmix
from ..parallel.tp_layers import ColumnParallelLinear, RowParallelLinear
from ..transformer.module import MegatronModule


def packed_tokens(t: torch.Tensor) -> torch.Tensor:
    """``[s, b, n]`` -> ``[b * s, n]`` with every sequence contiguous (a view when ``b == 1``)."""
    return t[:, 0] if t.shape[1] == 1 else t.transpose(0, 1).reshape(t.shape[0] * t.shape[1], t.shape[2])


def unpacked_tokens(t: torch.Tensor, s: int, b: int) -> torch.Tensor:
    return t.unsqueeze(1) if b == 1 else t.view(b, s, -1).transpose(0, 1).contiguous()


class GatedDeltaMixer(MegatronModule):
    def __init__(self, config, layer_number: int, num_heads: int, num_kv_heads: int, qk_dim: int, v_dim: int,
                 conv_taps: int, decay_rank: int, gate_rank: int, eps: float = None, unit_eps: float = 1e-6,
                 decay_per_head: bool = False, gate_act: str = "sigmoid"):
        super().__init__(config)
        if num_heads % num_kv_heads:
            raise ValueError("gated delta: heads must be a multiple of kv_heads")
        self.layer_number = layer_number
        self.nh, self.nkv, self.d, self.dv, self.taps = num_heads, num_kv_heads, qk_dim, v_dim, conv_taps
        self.decay_rank, self.gate_rank = int(decay_rank), int(gate_rank)
        self.decay_per_head, self.gate_act = bool(decay_per_head), gate_act
        self.eps = config.layernorm_epsilon if eps is None else eps
        self.unit_eps = unit_eps
        self.qk_ch, self.v_ch = num_kv_heads * qk_dim, num_heads * v_dim
        self.conv_ch = 2 * self.qk_ch + self.v_ch
        col = dict(config=config, init_method=config.init_method, bias=False, skip_bias_add=False, gather_output=False)
        self.decay_ch = num_heads if self.decay_per_head else num_heads * qk_dim
        self.a_rows, self.g_rows = self.decay_rank or self.decay_ch, self.gate_rank or self.v_ch
        self.in_proj = ColumnParallelLinear(config.hidden_size, self.conv_ch + self.a_rows + self.g_rows + num_heads, **col)
        self.decay_up = ColumnParallelLinear(decay_rank, self.decay_ch, **col) if self.decay_rank else None
        self.gate_up = ColumnParallelLinear(gate_rank, self.v_ch, **col) if self.gate_rank else None
        dev, dt_ = self.in_proj.weight.device, config.params_dtype
        self.conv_weight = nn.Parameter(torch.randn(self.conv_ch, conv_taps, device=dev).mul_(conv_taps ** -0.5).to(dt_))
        self.A_log = nn.Parameter(torch.zeros(num_heads, device=dev, dtype=dt_))
        self.dt_bias = nn.Parameter(torch.zeros(self.decay_ch, device=dev, dtype=dt_))
        self.norm_weight = nn.Parameter(torch.ones(v_dim, device=dev, dtype=dt_))
        self.out_proj = RowParallelLinear(self.v_ch, config.hidden_size, config=config,
                                          init_method=config.output_layer_init_method, bias=False, input_is_parallel=True,
                                          skip_bias_add=True)
        for p in (self.A_log, self.dt_bias):
            p._no_weight_decay = True

    def segments(self):
        """Row counts of the ``[q | k | v | a1 | g1 | b]`` segments of ``in_proj`` (``a1`` / ``g1`` are the full decay / gate rows
        when their rank is 0)."""
        return [("q", self.qk_ch), ("k", self.qk_ch), ("v", self.v_ch), ("a1", self.a_rows), ("g1", self.g_rows), ("b", self.nh)]

    def forward(self, hidden_states, inference_context=None, cache_index=None, **_):
        s, b = hidden_states.shape[0], hidden_states.shape[1]
        key = self.layer_number if cache_index is None else cache_index
        proj, _ = self.in_proj(hidden_states)
        proj = packed_tokens(proj)                                                     # [T, ...]
        qkv, a1, g1, braw = torch.split(proj, [self.conv_ch, self.a_rows, self.g_rows, self.nh], dim=-1)
        if inference_context is not None:
            if inference_context.is_static_batching():
                raise NotImplementedError("recurrent mixers serve through the dynamic engine")
            pb = inference_context.packed
            window = inference_context.recurrent_state(("delta.conv", key), (self.taps - 1, self.conv_ch),
                                                       proj.dtype)
            state = inference_context.recurrent_state(("delta.S", key), (self.nh, self.d, self.dv),
                                                      torch.float32)
        else:
            pb = seqmix.PackedBatch.dense(s, b, proj.device)
            window = proj.new_zeros(b, self.taps - 1, self.conv_ch)
            state = torch.zeros(b, self.nh, self.d, self.dv, dtype=torch.float32, device=proj.device)
        qkv = seqmix.causal_conv_silu(qkv, self.conv_weight, pb, window)
        T = qkv.shape[0]
        q, k, v = torch.split(qkv, [self.qk_ch, self.qk_ch, self.v_ch], dim=-1)
        dt = self.decay_up(a1.contiguous())[0] if self.decay_up is not None else a1
        log_decay, beta = seqmix.decay_gates(dt, braw, self.A_log, self.dt_bias)         # fp32 [T, H] or [T, H * d], [T, H]
        if not self.decay_per_head:
            log_decay = log_decay.view(T, self.nh, self.d)
        o = seqmix.delta_rule_scan(q.reshape(T, self.nkv, self.d), k.reshape(T, self.nkv, self.d),
                                   v.reshape(T, self.nh, self.dv), log_decay, beta, pb, state, self.unit_eps,
                                   self.d ** -0.5)
        gate = self.gate_up(g1.contiguous())[0] if self.gate_up is not None else g1
        y = seqmix.gated_head_rms_norm(o, self.norm_weight, gate, self.eps, proj.dtype, self.gate_act)
        return self.out_proj(unpacked_tokens(y, s, b))
