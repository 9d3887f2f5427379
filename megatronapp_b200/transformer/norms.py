"""LayerNorm / RMSNorm / L2Norm modules backed by the fused sm_100a norm kernel.

Parity: reference ``fusions/fused_layer_norm.py:30-169`` (``FusedLayerNorm``, zero-centred gamma,
``sequence_parallel`` attribute on the params) and ``transformer/torch_norm.py:9-96``.
"""
from __future__ import annotations

import torch
import torch.nn as nn

from .. import ops


class FusedLayerNorm(nn.Module):
    def __init__(self, config, hidden_size: int, eps: float = 1e-5, persist_layer_norm: bool = True,
                 zero_centered_gamma: bool = False, normalization: str = "LayerNorm"):
        super().__init__()
        self.config = config
        self.zero_centered_gamma = config.layernorm_zero_centered_gamma if config is not None else zero_centered_gamma
        self.normalization = config.normalization if config is not None else normalization
        if self.normalization not in ("LayerNorm", "RMSNorm"):
            raise ValueError(f"unsupported normalization {self.normalization}")
        self.eps = eps
        self.hidden_size = hidden_size
        dtype = config.params_dtype if config is not None else torch.float32
        dev = "cpu" if (config is None or config.use_cpu_initialization or not torch.cuda.is_available()) \
            else torch.cuda.current_device()
        init = 0.0 if self.zero_centered_gamma else 1.0
        self.weight = nn.Parameter(torch.full((hidden_size,), init, dtype=dtype, device=dev))
        if self.normalization == "LayerNorm":
            self.bias = nn.Parameter(torch.zeros(hidden_size, dtype=dtype, device=dev))
        else:
            self.register_parameter("bias", None)
        sp = bool(config.sequence_parallel) if config is not None else False
        setattr(self.weight, "sequence_parallel", sp)
        if self.bias is not None:
            setattr(self.bias, "sequence_parallel", sp)

    def forward(self, x):
        return ops.layer_norm(x, self.weight, self.bias, self.eps, rms=self.normalization == "RMSNorm",
                              zero_centered=self.zero_centered_gamma)


WrappedTorchNorm = FusedLayerNorm
LNImpl = FusedLayerNorm


class L2Norm(nn.Module):
    def __init__(self, hidden_size: int = 0, eps: float = 1e-6, **_):
        super().__init__()
        self.eps = eps

    def forward(self, x):
        xf = x.float()
        return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + self.eps)).type_as(x)


class IdentityOp(nn.Module):
    def __init__(self, *a, **k):
        super().__init__()

    def forward(self, x, *a, **k):
        return x


class IdentityFuncOp(IdentityOp):
    def forward(self, *a, **k):
        return super().forward


class ResidualRMSNorm(nn.Module):
    """RMS norm of an fp32 residual stream, fused with the addition that precedes it: ``forward(x, delta)`` adds
    ``delta`` (any dtype) into the fp32 ``x`` in place and returns ``(x, x / sqrt(mean(x^2) + eps) * weight)`` with the
    normalised copy in ``out_dtype`` (the dtype the following projections run in)."""

    def __init__(self, config, hidden_size: int, eps: float = 1e-5, out_dtype=None, weight_offset: float = 0.0):
        super().__init__()
        self.eps, self.hidden_size = eps, hidden_size
        self.weight_offset = float(weight_offset)     # 1.0: zero-centred weight, applied as 1 + w
        dtype = config.params_dtype if config is not None else torch.float32
        self.out_dtype = out_dtype          # None: the weight's dtype at call time
        dev = "cpu" if (config is None or config.use_cpu_initialization or not torch.cuda.is_available()) \
            else torch.cuda.current_device()
        self.weight = nn.Parameter(torch.full((hidden_size,), 1.0 - self.weight_offset, dtype=dtype, device=dev))
        setattr(self.weight, "sequence_parallel", bool(config.sequence_parallel) if config is not None else False)

    def forward(self, x, delta=None):
        from ..ops import seqmix

        shape = x.shape
        x2, y = seqmix.add_rms_norm(x.view(-1, shape[-1]), None if delta is None else delta.reshape(-1, shape[-1]),
                                    self.weight, self.eps, self.out_dtype or self.weight.dtype, self.weight_offset)
        return x2.view(shape), y.view(shape)


class BranchPair:
    """Outputs of two mixers that ran side by side on the same input, with the plain RMS-norm weight of each: the layer's
    result is ``(rms_norm(a) * weight_a + rms_norm(b) * weight_b) / 2``, which ``OutputRMSNormAdd`` computes inside its
    kernel."""

    def __init__(self, a, b, weight_a, weight_b):
        self.a, self.b, self.weight_a, self.weight_b = a, b, weight_a, weight_b


class OutputRMSNormAdd(nn.Module):
    """RMS norm of a sublayer's *output*, fused with the addition to the fp32 residual stream: ``forward(x, out)`` updates
    ``x += rms_norm(out) * (weight_offset + weight)`` in place and returns ``(x, x in out_dtype)``, the copy the next
    sublayer reads.  ``out`` may be a ``BranchPair``.  Statistics and the sum are fp32."""

    def __init__(self, config, hidden_size: int, eps: float = 1e-5, out_dtype=None, weight_offset: float = 0.0):
        super().__init__()
        self.eps, self.hidden_size, self.out_dtype = eps, hidden_size, out_dtype
        self.weight_offset = float(weight_offset)
        dtype = config.params_dtype if config is not None else torch.float32
        dev = "cpu" if (config is None or config.use_cpu_initialization or not torch.cuda.is_available()) \
            else torch.cuda.current_device()
        self.weight = nn.Parameter(torch.full((hidden_size,), 1.0 - self.weight_offset, dtype=dtype, device=dev))
        setattr(self.weight, "sequence_parallel", bool(config.sequence_parallel) if config is not None else False)

    def forward(self, x, out):
        from ..ops import seqmix

        shape, h = x.shape, x.shape[-1]
        dt = self.out_dtype or self.weight.dtype
        if isinstance(out, BranchPair):
            x2, y = seqmix.norm_add(x.view(-1, h), out.a.reshape(-1, h), self.weight, self.eps, dt, self.weight_offset,
                                    out.b.reshape(-1, h), out.weight_a, out.weight_b)
        else:
            x2, y = seqmix.norm_add(x.view(-1, h), out.reshape(-1, h), self.weight, self.eps, dt, self.weight_offset)
        return x2.view(shape), y.view(shape)


class ScaledPair:
    """Outputs of two mixers that ran side by side on the same input whose result is the weighted sum
    ``scale_a * (a + bias_a) + scale_b * b``; ``StreamConnection`` computes it inside its kernel, in fp32."""

    def __init__(self, a, b, bias_a=None, scale_a: float = 1.0, scale_b: float = 1.0):
        self.a, self.b, self.bias_a, self.scale_a, self.scale_b = a, b, bias_a, float(scale_a), float(scale_b)


class StreamUpdate:
    """A sublayer's output waiting to be written into the residual streams (by the next ``StreamConnection.read``)."""

    def __init__(self, out, conn: "StreamConnection"):
        self.out, self.conn = out, conn


class StreamConnection(nn.Module):
    """One sublayer's connection to ``streams`` fp32 residual streams ``x [.., S, W]`` (hyper-connections: Zhu et al.,
    "Hyper-Connections"), with the layer norm of the sublayer's input and an optional layer scale on its output::

        read:    u = sum_s inp[s] x_s;   h = layer_norm(u) * weight + bias
        write:   y = layer_scale * sublayer(h);   x_t <- sum_s mix[s, t] x_s + out[t] * y     (all t from the old streams)

    ``learned = False`` fixes ``inp = out = 1`` and ``mix = I``: with one stream this is the plain pre-norm residual layer,
    with several the read is the sum of the streams (used for the final norm).  The write is deferred: ``write(y)`` returns a
    ``StreamUpdate`` which the next ``read`` applies in the same kernel as its norm.  All arithmetic is fp32; ``h`` leaves in
    the parameter dtype."""

    def __init__(self, config, hidden_size: int, streams: int = 1, eps: float = 1e-5, learned: bool = True,
                 layer_scale: bool = False, bias: bool = True, center: bool = True, read_fill: float = 1.0):
        super().__init__()
        self.eps, self.hidden_size, self.streams, self.center = eps, hidden_size, int(streams), bool(center)
        dtype = config.params_dtype if config is not None else torch.float32
        dev = "cpu" if (config is None or config.use_cpu_initialization or not torch.cuda.is_available()) \
            else torch.cuda.current_device()
        self.weight = nn.Parameter(torch.ones(hidden_size, dtype=dtype, device=dev))
        self.bias = nn.Parameter(torch.zeros(hidden_size, dtype=dtype, device=dev)) if bias else None
        self.layer_scale = nn.Parameter(torch.ones(hidden_size, dtype=dtype, device=dev)) if layer_scale else None
        S = self.streams
        coef = dict(dtype=torch.float32, device=dev)
        tensors = (("inp", torch.full((S,), read_fill, **coef)), ("out", torch.ones(S, **coef)), ("mix", torch.eye(S, **coef)))
        for name, t in tensors:
            if learned:
                setattr(self, name, nn.Parameter(t))
            else:
                self.register_buffer(name, t, persistent=False)

    def read(self, x, update: "StreamUpdate" = None):
        """Apply ``update`` (if any) to the streams, then return ``(x, h)``: the streams and this sublayer's normed input."""
        return _stream_apply(x, update, self)

    def write(self, out) -> StreamUpdate:
        return StreamUpdate(out, self)


def _stream_apply(x, update, reader):
    """``x [s, b, S, W]`` or ``[T, S, W]``: the pending write of ``update`` and the read of ``reader`` in one kernel."""
    from ..ops import seqmix

    shape = x.shape
    S, W = shape[-2], shape[-1]
    x3 = x.view(-1, S, W)
    kw = {}
    if update is not None:
        o, c = update.out, update.conn
        if isinstance(o, ScaledPair):
            kw.update(a=o.a.reshape(-1, W), b=o.b.reshape(-1, W), bias_a=o.bias_a, scale_a=o.scale_a, scale_b=o.scale_b)
        else:
            kw.update(a=o.reshape(-1, W))
        kw.update(ls=c.layer_scale, mix=c.mix, outc=c.out)
    if reader is not None:
        kw.update(inp=reader.inp, weight=reader.weight, beta=reader.bias, eps=reader.eps, center=reader.center,
                  out_dtype=reader.weight.dtype)
    _, h = seqmix.stream_mix_norm(x3, **kw)
    return x, (None if h is None else h.view(*shape[:-2], W))
