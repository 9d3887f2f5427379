"""Grouped-query sliding-window attention with a linear distance penalty per head or a learned bias by distance bucket,
an optional sink in the softmax denominator, per-head RMS norm of queries and keys, and one scalar output gate per head.

Per token at position ``i``, from the mixer input ``x``::

    q, k   = W_q x + b_q, W_k x + b_k;   v = W_v x + b_v, or the projected keys themselves (``values_are_keys``)
    q, k   = rms_norm_per_head(q) * w_q, rms_norm_per_head(k) * w_k      (the values keep the un-normed keys)
    s_j    = q_h . k_kv(h)(j) * scale - slope_h * (i - j),   0 <= i - j < window
    p_j    = exp(s_j) / (sink + sum_j exp(s_j))                           sink 1: a key of score 0 without a value
    o_h    = sigmoid(w_g,h . x) * sum_j p_j v_kv(h)(j);   y = W_o concat(o) + b_o

``slope_h = 2^(-slope_exponent * (h + 1) / heads)`` (linear distance biases: Press, Smith and Lewis, "Train Short, Test Long:
Attention with Linear Biases Enables Input Length Extrapolation").  With ``bias_buckets = B`` a learned table
``rel_bias [B, heads]`` adds ``rel_bias[bucket(i - j), h]`` to the score instead (the scale does not multiply it): distances
below ``B / 2`` have a bucket each, larger ones share logarithmically spaced buckets up to ``bias_max``
(``distance_buckets``).  Positions enter in no other way.

The module follows the framework's other paged mixers: one fused input projection with the row segments
``[q | k | (v) | g]``, normed keys and values in the paged cache of the inference context, a row-parallel output projection.
Norm statistics, scores, weights and the weighted sum are fp32.  Every size and constant is a parameter.
"""
from __future__ import annotations

import math
from typing import Optional

import torch
import torch.nn as nn

from ..ops import seqmix
from ..parallel.tp_layers import ColumnParallelLinear, RowParallelLinear
from ..ssm.gated_delta import packed_tokens, unpacked_tokens
from .mixed_head_attention import dense_pages
from .module import MegatronModule


def distance_slopes(num_heads: int, exponent: float = 8.0) -> torch.Tensor:
    """``2^(-exponent * (h + 1) / num_heads)`` for ``h = 0 .. num_heads - 1`` (computed in fp64, returned as fp32)."""
    h = torch.arange(1, num_heads + 1, dtype=torch.float64)
    return torch.pow(torch.tensor(2.0, dtype=torch.float64), -exponent * h / num_heads).float()


def distance_buckets(num_buckets: int, bias_max: float, length: int) -> torch.Tensor:
    """Bucket of every distance ``n = 0 .. length - 1`` (int64).  With ``half = num_buckets // 2``: ``n`` itself below ``half``,
    else ``min(num_buckets - 1, half + floor(ln(n / half) / ln(bias_max / half) * (num_buckets - half)))``; computed in fp64."""
    half = num_buckets // 2
    n = torch.arange(length, dtype=torch.float64)
    if half < 1 or bias_max <= half:
        return n.clamp(max=num_buckets - 1).long()
    far = half + torch.floor(torch.log(n.clamp(min=half) / half) / math.log(bias_max / half) * (num_buckets - half))
    return torch.where(n < half, n, far.clamp(max=num_buckets - 1)).long()


class WindowAttention(MegatronModule):
    def __init__(self, config, layer_number: int, num_heads: int, num_kv_heads: int, qk_dim: int, v_dim: int, softmax_scale: float,
                 window: int = 0, sink: bool = False, slope_exponent: Optional[float] = 8.0, qk_norm: bool = True,
                 values_are_keys: bool = False, head_gate: bool = True, bias: bool = True, eps: Optional[float] = None,
                 output_scale: float = 1.0, bias_buckets: int = 0, bias_max: float = 0.0):
        super().__init__(config)
        if num_heads % num_kv_heads:
            raise ValueError("window attention: heads must be a multiple of kv_heads")
        if values_are_keys and v_dim != qk_dim:
            raise ValueError("window attention: values that are the keys need vdim == dim")
        self.layer_number = layer_number
        self.nh, self.nkv, self.d, self.dv = num_heads, num_kv_heads, qk_dim, v_dim
        self.window, self.sink, self.softmax_scale, self.output_scale = int(window), bool(sink), float(softmax_scale), float(output_scale)
        self.values_are_keys, self.qk_norm = bool(values_are_keys), bool(qk_norm)
        self.eps = config.layernorm_epsilon if eps is None else eps
        self.q_ch, self.k_ch, self.o_ch = num_heads * qk_dim, num_kv_heads * qk_dim, num_heads * v_dim
        self.v_ch = 0 if values_are_keys else num_kv_heads * v_dim
        self.g_ch = num_heads if head_gate else 0
        self.in_proj = ColumnParallelLinear(config.hidden_size, self.q_ch + self.k_ch + self.v_ch + self.g_ch, config=config,
                                            init_method=config.init_method, bias=bias, skip_bias_add=False, gather_output=False)
        dev, dt_ = self.in_proj.weight.device, config.params_dtype
        if qk_norm:
            self.q_norm_weight = nn.Parameter(torch.ones(qk_dim, device=dev, dtype=dt_))
            self.k_norm_weight = nn.Parameter(torch.ones(qk_dim, device=dev, dtype=dt_))
        self.register_buffer("slopes", distance_slopes(num_heads, slope_exponent).to(dev) if slope_exponent is not None else None,
                             persistent=False)
        self.bias_buckets, self.bias_max = int(bias_buckets), float(bias_max)
        if self.bias_buckets:
            self.rel_bias = nn.Parameter(torch.zeros(self.bias_buckets, num_heads, device=dev, dtype=dt_))
        self._dist_bias = None                                     # (version, table): the bias by distance, fp32 [L, H]
        self.out_proj = RowParallelLinear(self.o_ch, config.hidden_size, config=config, init_method=config.output_layer_init_method,
                                          bias=bias, input_is_parallel=True, skip_bias_add=True)

    def segments(self):
        """Row counts of the ``[q | k | v | g]`` segments of ``in_proj`` (absent segments are left out)."""
        return [(n, c) for n, c in (("q", self.q_ch), ("k", self.k_ch), ("v", self.v_ch), ("g", self.g_ch)) if c]

    def distance_bias(self) -> Optional[torch.Tensor]:
        """The learned bias laid out by distance, fp32 ``[L, heads]``: one row per distance the window lets through, or, without
        a window, up to the distance from which every key falls into the last bucket.  Rebuilt when the table changes."""
        if not self.bias_buckets:
            return None
        w = self.rel_bias
        tag = (w._version, w.data_ptr(), w.device)
        if self._dist_bias is None or self._dist_bias[0] != tag:
            sat = int(math.ceil(max(self.bias_max, self.bias_buckets))) + 1           # every distance >= sat - 1 is in the last bucket
            length = min(self.window, sat) if self.window > 0 else sat
            idx = distance_buckets(self.bias_buckets, self.bias_max, length).to(w.device)
            self._dist_bias = (tag, w.detach().float()[idx].contiguous())
        return self._dist_bias[1]

    def forward(self, hidden_states, inference_context=None, cache_index=None, **_):
        s, b = hidden_states.shape[0], hidden_states.shape[1]
        key = self.layer_number if cache_index is None else cache_index
        proj, _ = self.in_proj(hidden_states)
        proj = packed_tokens(proj)                                                     # [T, q | k | (v) | g]
        T = proj.shape[0]
        q = proj[:, :self.q_ch].view(T, self.nh, self.d)
        k = proj[:, self.q_ch:self.q_ch + self.k_ch].view(T, self.nkv, self.d)
        v = k if self.values_are_keys else proj[:, self.q_ch + self.k_ch:self.q_ch + self.k_ch + self.v_ch].view(T, self.nkv, self.dv)
        gate = proj[:, proj.shape[1] - self.g_ch:] if self.g_ch else None
        if self.qk_norm:
            q, kn = seqmix.head_rms_norm(q, self.q_norm_weight, self.eps), seqmix.head_rms_norm(k, self.k_norm_weight, self.eps)
        else:
            kn = k
        ctx = inference_context
        if ctx is not None:
            if ctx.is_static_batching():
                raise NotImplementedError("window attention serves through the dynamic (paged) engine")
            o = ctx.attend_window(key, q, kn, v, self.softmax_scale, self.window, self.slopes, self.sink, gate, self.output_scale,
                                  self.distance_bias())
        else:
            table, tok_req, tok_len = dense_pages(s, b, proj.device)
            o = seqmix.window_attention_paged(q, kn.contiguous(), v.contiguous(), table, tok_req, tok_len, s, self.softmax_scale,
                                              self.window, self.slopes, self.sink, gate, self.output_scale,
                                              dist_bias=self.distance_bias())
        return self.out_proj(unpacked_tokens(o, s, b))
