"""Layers over an fp32 residual stream with an arbitrary sequence mixer, and the blocks that stack them: pre-norm
(``ResidualF32Layer`` / ``ResidualF32Block``), norm on the sublayer's output (``OutputNormF32Layer`` /
``OutputNormF32Block``), several streams (``StreamLayer`` / ``StreamBlock``) and one norm read by mixer and feed-forward side
by side (``ParallelF32Layer`` / ``ParallelF32Block``), further down.

``x <- x + mixer(norm1(x));  x <- x + mlp(norm2(x))`` (the second half is absent for a layer without feed-forward).
The stream ``x`` stays fp32 whatever the parameter dtype; every addition is fused into the norm that follows it
(``ResidualRMSNorm``), so a layer hands ``(x, pending)`` to the next one and the block's final norm performs the last
addition.  The mixer is any module with the ``forward(hidden_states, inference_context=, cross_layer=) -> (out, bias)``
contract of the framework's attention and recurrent mixers; layers of one block may differ in every size.
"""
from __future__ import annotations

from typing import Callable, List, Optional

import torch
import torch.nn as nn

from ..scan.tracer import scope as _scope
from .module import MegatronModule
from .norms import BranchPair, OutputRMSNormAdd, ResidualRMSNorm


class ResidualF32Layer(MegatronModule):
    def __init__(self, config, layer_number: int, mixer: nn.Module, mlp: Optional[nn.Module] = None):
        super().__init__(config)
        self.layer_number = layer_number
        eps = config.layernorm_epsilon
        self.input_layernorm = ResidualRMSNorm(config, config.hidden_size, eps)
        self.mixer = mixer
        self.mlp = mlp
        self.pre_mlp_layernorm = ResidualRMSNorm(config, config.hidden_size, eps) if mlp is not None else None
        if mlp is not None and hasattr(mlp, "set_layer_number"):
            mlp.set_layer_number(layer_number)

    def forward(self, x, pending=None, inference_context=None, cross_layer=None):
        with _scope("transformer_layer", layer=self.layer_number):
            x, h = self.input_layernorm(x, pending)
            out, bias = self.mixer(h, inference_context=inference_context, cross_layer=cross_layer)
            if bias is not None:
                out = out + bias
            if self.mlp is None:
                return x, out
            x, h = self.pre_mlp_layernorm(x, out)
            out, bias = self.mlp(h)
            if bias is not None:
                out = out + bias
        return x, out


class ResidualF32Block(MegatronModule):
    """A stack of ``ResidualF32Layer`` followed by the final norm.  ``layer_builders[i](layer_number)`` returns layer
    ``i``; ``tap`` (optional callable) receives ``(layer_index, residual_after_layer)`` for inspection tools."""

    def __init__(self, config, layer_builders: List[Callable[[int], ResidualF32Layer]], post_process: bool = True):
        super().__init__(config)
        self.layers = nn.ModuleList([build(i) for i, build in enumerate(layer_builders)])
        self.final_layernorm = ResidualRMSNorm(config, config.hidden_size, config.layernorm_epsilon) if post_process else None
        self.input_tensor = None
        self.tap = None

    def set_input_tensor(self, t):
        self.input_tensor = t

    def forward(self, hidden_states, inference_context=None):
        x = hidden_states if self.input_tensor is None else self.input_tensor
        if x.dtype != torch.float32:
            x = x.float()
        pending, cross_layer = None, {}
        for i, layer in enumerate(self.layers):
            x, pending = layer(x, pending, inference_context=inference_context, cross_layer=cross_layer)
            if self.tap is not None:
                self.tap(i, x + pending.float())
        if self.final_layernorm is None:
            return x + pending.float()
        _, h = self.final_layernorm(x, pending)
        return h


class OutputNormF32Layer(MegatronModule):
    """``x <- x + norm1(mixer(x));  x <- x + norm2(mlp(x))``: the sublayers read the stream itself, only their outputs are
    normed (``OutputRMSNormAdd``, whose kernel also performs the addition and hands out the copy of ``x`` in the
    activation dtype that the next sublayer reads).  ``cache_index`` names the cache / state a call uses, so that one
    layer object can run at several depths of a block, each with a cache of its own."""

    def __init__(self, config, layer_number: int, mixer: nn.Module, mlp: Optional[nn.Module] = None, weight_offset: float = 0.0):
        super().__init__(config)
        self.layer_number = layer_number
        eps = config.layernorm_epsilon
        self.mixer, self.mlp = mixer, mlp
        self.mixer_norm = OutputRMSNormAdd(config, config.hidden_size, eps, weight_offset=weight_offset)
        self.mlp_norm = OutputRMSNormAdd(config, config.hidden_size, eps, weight_offset=weight_offset) if mlp is not None else None
        if mlp is not None and hasattr(mlp, "set_layer_number"):
            mlp.set_layer_number(layer_number)

    def forward(self, x, h, inference_context=None, cache_index=None):
        with _scope("transformer_layer", layer=self.layer_number):
            out, bias = self.mixer(h, inference_context=inference_context,
                                   cache_index=self.layer_number if cache_index is None else cache_index)
            if bias is not None:
                out = out + bias
            x, h = self.mixer_norm(x, out)
            if self.mlp is not None:
                out, bias = self.mlp(h)
                if bias is not None:
                    out = out + bias
                x, h = self.mlp_norm(x, out)
        return x, h


class OutputNormF32Block(MegatronModule):
    """A stack of ``OutputNormF32Layer`` runs followed by the final norm.  ``layer_builders[i](i)`` builds layer object
    ``i``; ``runs`` lists, depth by depth, which object runs there (default: each once, in order), so a layer's weights
    can serve several depths.  Run ``k`` uses cache / state index ``k``.  ``tap(run, residual)`` as in ``ResidualF32Block``."""

    def __init__(self, config, layer_builders: List[Callable[[int], OutputNormF32Layer]], runs: Optional[List[int]] = None,
                 post_process: bool = True, weight_offset: float = 0.0):
        super().__init__(config)
        self.layers = nn.ModuleList([build(i) for i, build in enumerate(layer_builders)])
        self.runs = list(range(len(self.layers))) if runs is None else [int(r) for r in runs]
        if any(not 0 <= r < len(self.layers) for r in self.runs):
            raise ValueError("a run names a layer that does not exist")
        self.final_layernorm = ResidualRMSNorm(config, config.hidden_size, config.layernorm_epsilon,
                                               weight_offset=weight_offset) if post_process else None
        self.input_tensor = None
        self.tap = None

    def set_input_tensor(self, t):
        self.input_tensor = t

    def forward(self, hidden_states, inference_context=None):
        x = hidden_states if self.input_tensor is None else self.input_tensor
        if x.dtype != torch.float32:
            x = x.float()
        dt = self.config.params_dtype
        h = x if dt == torch.float32 else x.to(dt)
        for k, r in enumerate(self.runs):
            x, h = self.layers[r](x, h, inference_context=inference_context, cache_index=k)
            if self.tap is not None:
                self.tap(k, x)
        if self.final_layernorm is None:
            return x
        _, y = self.final_layernorm(x, None)
        return y


class StreamLayer(MegatronModule):
    """Pre-norm layer over ``streams`` fp32 residual streams: each sublayer reads a weighted sum of the streams through its
    layer norm and writes its (layer-scaled) output back into all of them (``norms.StreamConnection``).  With
    ``learned_connections = False`` and one stream it is ``x <- x + ls1 * mixer(norm1(x)); x <- x + ls2 * mlp(norm2(x))``.
    A sublayer's write is handed on as a ``StreamUpdate`` and fused into the next sublayer's read.  ``cache_index`` names the
    cache / state a call uses, so one layer object can run at several depths of a block."""

    def __init__(self, config, layer_number: int, mixer: nn.Module, mlp: Optional[nn.Module] = None, streams: int = 1,
                 learned_connections: bool = True, layer_scale: bool = False):
        super().__init__(config)
        from .norms import StreamConnection

        self.layer_number = layer_number
        eps, W = config.layernorm_epsilon, config.hidden_size
        self.mixer, self.mlp = mixer, mlp
        self.mixer_conn = StreamConnection(config, W, streams, eps, learned_connections, layer_scale)
        self.mlp_conn = StreamConnection(config, W, streams, eps, learned_connections, layer_scale) if mlp is not None else None
        if mlp is not None and hasattr(mlp, "set_layer_number"):
            mlp.set_layer_number(layer_number)

    def forward(self, x, pending=None, inference_context=None, cache_index=None):
        with _scope("transformer_layer", layer=self.layer_number):
            x, h = self.mixer_conn.read(x, pending)
            out, bias = self.mixer(h, inference_context=inference_context,
                                   cache_index=self.layer_number if cache_index is None else cache_index)
            if bias is not None:
                out = out + bias
            pending = self.mixer_conn.write(out)
            if self.mlp is not None:
                x, h = self.mlp_conn.read(x, pending)
                out, bias = self.mlp(h)
                if bias is not None:
                    out = out + bias
                pending = self.mlp_conn.write(out)
        return x, pending


class StreamBlock(MegatronModule):
    """A stack of ``StreamLayer`` runs followed by the final layer norm of the sum of the streams.  ``layer_builders[i](i)``
    builds layer object ``i``; ``runs`` lists, depth by depth, which object runs there (default: each once, in order), so a
    span of layers can be repeated with the same weights; run ``k`` uses cache / state index ``k``.  The streams all start as
    copies of the block's input.  ``tap(run, sum of the streams)`` receives the residual after every run."""

    def __init__(self, config, layer_builders: List[Callable[[int], StreamLayer]], runs: Optional[List[int]] = None,
                 streams: int = 1, post_process: bool = True):
        super().__init__(config)
        from .norms import StreamConnection

        self.layers = nn.ModuleList([build(i) for i, build in enumerate(layer_builders)])
        self.runs = list(range(len(self.layers))) if runs is None else [int(r) for r in runs]
        if any(not 0 <= r < len(self.layers) for r in self.runs):
            raise ValueError("a run names a layer that does not exist")
        self.streams = int(streams)
        self.final_layernorm = StreamConnection(config, config.hidden_size, streams, config.layernorm_epsilon,
                                                learned=False) if post_process else None
        self.input_tensor = None
        self.tap = None

    def set_input_tensor(self, t):
        self.input_tensor = t

    def forward(self, hidden_states, inference_context=None):
        from .norms import _stream_apply

        x = hidden_states if self.input_tensor is None else self.input_tensor
        if x.dtype != torch.float32:
            x = x.float()
        if x.dim() == 3:                                            # [s, b, W]: every stream starts as the embedding output
            x = x.unsqueeze(-2).repeat(1, 1, self.streams, 1)
        pending = None
        for k, r in enumerate(self.runs):
            x, pending = self.layers[r](x, pending, inference_context=inference_context, cache_index=k)
            if self.tap is not None:
                x, _ = _stream_apply(x, pending, None)
                pending = None
                self.tap(k, x.sum(-2))
        if self.final_layernorm is None:
            x, _ = _stream_apply(x, pending, None) if pending is not None else (x, None)
            return x
        _, y = self.final_layernorm.read(x, pending)
        return y


class ParallelF32Layer(MegatronModule):
    """One norm, two sublayers that both read it, one addition::

        h = norm(x);   x <- x + mixer(h + conv(h)) + mlp(h);   x <- x + rms_norm(side(x, e)) * w_side

    ``conv`` (``input_conv_taps > 1``) is a depth-wise causal convolution over time on the mixer's input only, its last
    ``taps - 1`` inputs kept per sequence in the inference context's state rows; ``token_side`` (optional,
    ``embeddings.TokenSideInput``) brings in the token's vector ``e`` for this layer after the feed-forward.  The stream ``x`` is
    fp32.  The additions run in ``ops.seqmix.norm_add``: the first takes the mixer's output (a ``BranchPair`` of two mixers is
    normed and averaged there), the feed-forward's output, and hands out ``x`` in the activation dtype for the side input; the
    last one also computes the next layer's norm, so a layer receives ``(x, h)`` and returns ``(x, h_next)``."""

    def __init__(self, config, layer_number: int, mixer: nn.Module, mlp: Optional[nn.Module] = None, input_conv_taps: int = 0,
                 token_side: Optional[nn.Module] = None):
        super().__init__(config)
        self.layer_number = layer_number
        W, eps = config.hidden_size, config.layernorm_epsilon
        self.eps = eps
        self.input_layernorm = ResidualRMSNorm(config, W, eps)
        self.mixer, self.mlp, self.token_side = mixer, mlp, token_side
        self.taps = int(input_conv_taps)
        if self.taps > 1:
            dev = self.input_layernorm.weight.device
            self.input_conv_weight = nn.Parameter(torch.zeros(W, self.taps, dtype=config.params_dtype, device=dev))
        if mlp is not None and hasattr(mlp, "set_layer_number"):
            mlp.set_layer_number(layer_number)

    def mixer_input(self, h, inference_context, key):
        """``h + conv(h)`` over time, ``h [s, b, W]``."""
        from ..ops import seqmix
        from ..ssm.gated_delta import packed_tokens, unpacked_tokens

        if self.taps <= 1:
            return h
        s, b = h.shape[0], h.shape[1]
        hp = packed_tokens(h)
        if inference_context is not None:
            if inference_context.is_static_batching():
                raise NotImplementedError("layers with an input convolution serve through the dynamic engine")
            pb = inference_context.packed
            window = inference_context.recurrent_state(("layer.conv", key), (self.taps - 1, h.shape[-1]), h.dtype)
        else:
            pb = seqmix.PackedBatch.dense(s, b, h.device)
            window = h.new_zeros(b, self.taps - 1, h.shape[-1])
        return unpacked_tokens(seqmix.causal_conv(hp, self.input_conv_weight, pb, window, residual=True), s, b)

    def forward(self, x, h, inference_context=None, cache_index=None, side=None, next_weight=None):
        from ..ops import seqmix

        key = self.layer_number if cache_index is None else cache_index
        W = x.shape[-1]
        with _scope("transformer_layer", layer=self.layer_number):
            out, bias = self.mixer(self.mixer_input(h, inference_context, key), inference_context=inference_context, cache_index=key)
            if bias is not None:
                out = out + bias
            ff = None
            if self.mlp is not None:
                ff, fb = self.mlp(h)
                ff = (ff if fb is None else ff + fb).reshape(-1, W)
            x2 = x.view(-1, W)
            last = self.token_side is None
            kw = dict(extra=ff, next_weight=next_weight if last else None)
            if isinstance(out, BranchPair):
                _, y = seqmix.norm_add(x2, out.a.reshape(-1, W), None, self.eps, h.dtype, 0.0, out.b.reshape(-1, W), out.weight_a,
                                       out.weight_b, **kw)
            else:
                _, y = seqmix.norm_add(x2, out.reshape(-1, W), None, self.eps, h.dtype, **kw)
            if not last:
                if side is None:
                    raise ValueError("this layer takes a per-token side input")
                from ..ssm.gated_delta import packed_tokens, unpacked_tokens

                s, b = x.shape[0], x.shape[1]
                d = unpacked_tokens(self.token_side(packed_tokens(y.view(x.shape)), side), s, b)
                _, y = seqmix.norm_add(x2, d.reshape(-1, W), self.token_side.norm_weight, self.token_side.eps, h.dtype,
                                       next_weight=next_weight)
        return x, y.view(x.shape)


class ParallelF32Block(MegatronModule):
    """A stack of ``ParallelF32Layer`` runs followed by the final RMS norm.  ``layer_builders[i](i)`` builds layer object ``i``;
    ``runs`` lists, depth by depth, which object runs there (default: each once, in order); run ``k`` uses cache / state index
    ``k``.  ``side_slice(rows, layer)`` (optional) cuts a layer's part out of the per-token side rows given to ``forward``.
    ``tap(run, residual)`` receives the stream after every run."""

    def __init__(self, config, layer_builders: List[Callable[[int], ParallelF32Layer]], runs: Optional[List[int]] = None,
                 post_process: bool = True, side_slice: Optional[Callable] = None):
        super().__init__(config)
        self.layers = nn.ModuleList([build(i) for i, build in enumerate(layer_builders)])
        self.runs = list(range(len(self.layers))) if runs is None else [int(r) for r in runs]
        if any(not 0 <= r < len(self.layers) for r in self.runs):
            raise ValueError("a run names a layer that does not exist")
        self.final_layernorm = ResidualRMSNorm(config, config.hidden_size, config.layernorm_epsilon) if post_process else None
        self.side_slice = side_slice
        self.input_tensor = None
        self.tap = None

    def set_input_tensor(self, t):
        self.input_tensor = t

    def forward(self, hidden_states, inference_context=None, side=None):
        x = hidden_states if self.input_tensor is None else self.input_tensor
        if x.dtype != torch.float32:
            x = x.float()
        if not self.runs:
            return x if self.final_layernorm is None else self.final_layernorm(x, None)[1]
        _, h = self.layers[self.runs[0]].input_layernorm(x, None)
        n = len(self.runs)
        for k, r in enumerate(self.runs):
            nxt = self.layers[self.runs[k + 1]].input_layernorm.weight if k + 1 < n else (
                self.final_layernorm.weight if self.final_layernorm is not None else None)
            e = self.side_slice(side, r) if (side is not None and self.side_slice is not None) else side
            x, h = self.layers[r](x, h, inference_context=inference_context, cache_index=k, side=e, next_weight=nxt)
            if self.tap is not None:
                self.tap(k, x)
        return x if self.final_layernorm is None else h
