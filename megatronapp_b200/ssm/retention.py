"""Retention mixer: linear attention with a fixed decay per head and neither softmax nor denominator (Sun et al.,
"Retentive Network: A Successor to Transformer for Large Language Models").

Per head a matrix memory ``S [d, dv]`` is carried from token to token::

    q, k = rot(W_q h), rot(W_k h) * d^-1/2;   v = W_v h
    S <- decay_h * S + k v^T;   o = S^T q
    y = W_o (concat_h(o_h / rms(o_h)) * silu(W_g h))

``rot`` turns the first ``rot_dims`` dimensions of every head by the token's position, dimension ``i`` paired with
``i + rot_dims / 2`` and the angle ``position * rot_base^(-2 i / rot_dims)``; the other dimensions pass unchanged.  The decays
are constants of the model (``decays``, one per head), not weights.

The module keeps the shape of the framework's other recurrent mixers (``ssm/gated_delta.py``): one fused input projection
whose rows are the segments ``[q | k | v | g]``, the fp32 memory of every sequence in the inference context's state rows (so
prompts may arrive whole, in portions or token by token), a row-parallel output projection.  Angles, the rotated q and k,
the memory and the read-out's norm are fp32 whatever the parameter dtype.
"""
from __future__ import annotations

from typing import Optional, Sequence

import torch

from ..ops import seqmix
from ..parallel.tp_layers import ColumnParallelLinear, RowParallelLinear
from ..transformer.module import MegatronModule
from .gated_delta import packed_tokens, unpacked_tokens


class RetentionMixer(MegatronModule):
    def __init__(self, config, layer_number: int, num_heads: int, qk_dim: int, v_dim: int, decays: Sequence[float],
                 rot_dims: int = 0, rot_base: float = 10000.0, eps: Optional[float] = None, key_scale: Optional[float] = None):
        super().__init__(config)
        if len(decays) != num_heads:
            raise ValueError(f"retention: {len(decays)} decays for {num_heads} heads")
        if rot_dims % 2 or rot_dims > qk_dim:
            raise ValueError("retention: rot_dims must be even and at most the head size")
        self.layer_number = layer_number
        self.nh, self.d, self.dv, self.rot_dims, self.rot_base = num_heads, qk_dim, v_dim, int(rot_dims), float(rot_base)
        self.eps = config.layernorm_epsilon if eps is None else eps
        self.key_scale = qk_dim ** -0.5 if key_scale is None else float(key_scale)
        self.qk_ch, self.v_ch = num_heads * qk_dim, num_heads * v_dim
        self.in_proj = ColumnParallelLinear(config.hidden_size, 2 * self.qk_ch + 2 * self.v_ch, config=config,
                                            init_method=config.init_method, bias=False, skip_bias_add=False, gather_output=False)
        dev = self.in_proj.weight.device
        self.register_buffer("decays", torch.tensor([float(x) for x in decays], dtype=torch.float32, device=dev), persistent=False)
        self.register_buffer("inv_freq", seqmix.rotary_frequencies(self.rot_dims, self.rot_base, dev), persistent=False)
        self.out_proj = RowParallelLinear(self.v_ch, config.hidden_size, config=config, init_method=config.output_layer_init_method,
                                          bias=False, input_is_parallel=True, skip_bias_add=True)

    def segments(self):
        """Row counts of the ``[q | k | v | g]`` segments of ``in_proj``."""
        return [("q", self.qk_ch), ("k", self.qk_ch), ("v", self.v_ch), ("g", self.v_ch)]

    def forward(self, hidden_states, inference_context=None, cache_index=None, **_):
        s, b = hidden_states.shape[0], hidden_states.shape[1]
        key = self.layer_number if cache_index is None else cache_index
        proj, _ = self.in_proj(hidden_states)
        proj = packed_tokens(proj)                                                     # [T, q | k | v | g]
        T = proj.shape[0]
        q, k, v, gate = torch.split(proj, [n for _, n in self.segments()], dim=-1)
        if inference_context is not None:
            if inference_context.is_static_batching():
                raise NotImplementedError("recurrent mixers serve through the dynamic engine")
            pb, positions = inference_context.packed, inference_context.positions
            state = inference_context.recurrent_state(("retention.S", key), (self.nh, self.d, self.dv), torch.float32)
        else:
            pb = seqmix.PackedBatch.dense(s, b, proj.device)
            positions = torch.arange(s, device=proj.device).repeat(b)
            state = torch.zeros(b, self.nh, self.d, self.dv, dtype=torch.float32, device=proj.device)
        o = seqmix.retention_scan(q.view(T, self.nh, self.d), k.view(T, self.nh, self.d), v.view(T, self.nh, self.dv), self.decays,
                                  pb, state, positions if self.inv_freq is not None else None, self.inv_freq, self.key_scale)
        y = seqmix.gated_head_rms_norm(o, None, gate, self.eps, proj.dtype, "silu")
        return self.out_proj(unpacked_tokens(y, s, b))
