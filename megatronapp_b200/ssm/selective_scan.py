"""Selective-scan mixer (Gu and Dao, "Mamba: Linear-Time Sequence Modeling with Selective State Spaces"): one decay per
channel and state, a step size per channel from a low-rank projection.

Per token, from the mixer input ``h``::

    [x | z]      = W_in h;    x = silu(causal_conv(x) + b_conv)                    depth-wise, ``taps`` wide
    [dt | B | C] = W_x x;     dt = softplus(W_dt dt + b_dt)                        one step size per channel
    S[c, n] <- exp(-dt_c exp(A_log[c, n])) S[c, n] + dt_c x_c B_n;   y_c = sum_n S[c, n] C_n + D_c x_c
    out = W_o (y * silu(z))

The module keeps the shape of the framework's other recurrent mixers (``ssm/mamba.py``, ``ssm/gated_delta.py``): the
convolution window (the last ``taps - 1`` inputs) and the fp32 state ``[inner, state]`` of every sequence live in the
inference context's state rows, so prompts may arrive whole, in portions or token by token.  Step sizes (the low-rank
projection's output included), decays and the state are fp32 whatever the parameter dtype.
"""
from __future__ import annotations

import torch
import torch.nn as nn

from .. import ops
from ..ops import seqmix
from ..parallel.tp_layers import ColumnParallelLinear, RowParallelLinear
from ..transformer.module import MegatronModule
from .gated_delta import packed_tokens, unpacked_tokens


class SelectiveScanMixer(MegatronModule):
    def __init__(self, config, layer_number: int, inner: int, state: int, dt_rank: int, conv_taps: int = 4, output_scale: float = 1.0):
        super().__init__(config)
        self.layer_number = layer_number
        self.inner, self.n_state, self.dt_rank, self.taps, self.output_scale = inner, state, dt_rank, max(1, int(conv_taps)), float(output_scale)
        col = dict(config=config, init_method=config.init_method, bias=False, skip_bias_add=False, gather_output=False)
        self.in_proj = ColumnParallelLinear(config.hidden_size, 2 * inner, **col)
        self.x_proj = ColumnParallelLinear(inner, dt_rank + 2 * state, **col)
        dev, dt_ = self.in_proj.weight.device, config.params_dtype
        self.conv_weight = nn.Parameter(torch.randn(inner, self.taps, device=dev).mul_(self.taps ** -0.5).to(dt_))
        self.conv_bias = nn.Parameter(torch.zeros(inner, device=dev, dtype=dt_))
        self.dt_weight = nn.Parameter(torch.randn(inner, dt_rank, device=dev).mul_(dt_rank ** -0.5).to(dt_))
        self.dt_bias = nn.Parameter(torch.zeros(inner, device=dev, dtype=dt_))
        self.A_log = nn.Parameter(torch.log(torch.arange(1, state + 1, dtype=torch.float32, device=dev)).repeat(inner, 1).to(dt_))
        self.D = nn.Parameter(torch.ones(inner, device=dev, dtype=dt_))
        self.out_proj = RowParallelLinear(inner, config.hidden_size, config=config, init_method=config.output_layer_init_method,
                                          bias=False, input_is_parallel=True, skip_bias_add=True)
        for p in (self.A_log, self.D, self.dt_bias):
            p._no_weight_decay = True

    def step_sizes(self, dt_low: torch.Tensor) -> torch.Tensor:
        """``W_dt dt_low`` as fp32 ``[T, inner]`` (the bias and the softplus belong to the scan kernel)."""
        if (dt_low.is_cuda and dt_low.dtype != torch.float32 and self.dt_rank % 8 == 0 and dt_low.stride(0) % 8 == 0
                and self.inner % 4 == 0 and dt_low.data_ptr() % 16 == 0):
            return ops.gemm(dt_low, self.dt_weight, epilogue=ops.EPI_STORE_F32)      # 16-bit operands, fp32 accumulator stored as is
        return dt_low.float() @ self.dt_weight.float().t()

    def forward(self, hidden_states, inference_context=None, cache_index=None, **_):
        s, b = hidden_states.shape[0], hidden_states.shape[1]
        key = self.layer_number if cache_index is None else cache_index
        xz, _ = self.in_proj(hidden_states)
        xz = packed_tokens(xz)                                                         # [T, x | z]
        x, z = xz[:, :self.inner], xz[:, self.inner:]
        if inference_context is not None:
            if inference_context.is_static_batching():
                raise NotImplementedError("recurrent mixers serve through the dynamic engine")
            pb = inference_context.packed
            window = inference_context.recurrent_state(("selscan.conv", key), (self.taps - 1, self.inner), xz.dtype)
            state = inference_context.recurrent_state(("selscan.S", key), (self.inner, self.n_state), torch.float32)
        else:
            pb = seqmix.PackedBatch.dense(s, b, xz.device)
            window = xz.new_zeros(b, self.taps - 1, self.inner)
            state = torch.zeros(b, self.inner, self.n_state, dtype=torch.float32, device=xz.device)
        x = seqmix.causal_conv_silu(x, self.conv_weight, pb, window, self.conv_bias)
        dbc, _ = self.x_proj(x.unsqueeze(1))
        dbc = dbc[:, 0]
        R, N = self.dt_rank, self.n_state
        dt_pre = self.step_sizes(dbc[:, :R])
        y = seqmix.selective_scan(x, dt_pre, dbc[:, R:R + N], dbc[:, R + N:], self.A_log, self.D, pb, state, z, self.dt_bias,
                                  self.output_scale)
        return self.out_proj(unpacked_tokens(y, s, b))
