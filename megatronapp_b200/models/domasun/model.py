"""Domasun: a decoder-only hybrid.  Word embedding plus sinusoidal positions; pre-norm layers (layer norm with bias, layer
scale on every sublayer's output) over several fp32 residual streams joined by hyper-connections; every mixer is a
sliding-window attention (values are the un-normed keys, per-head q / k RMS norm, linear distance penalty, a sink in the
softmax denominator, one output gate per head) side by side with a selective scan, their results added with fixed weights; a
mixture of clamped gated experts with a gated shared expert; a span of layers may run several times in a row with the same
weights and a cache per pass; the logits are soft-capped.

Assembled from the framework's parts: ``LanguageModelEmbedding`` (sinusoidal), ``StreamBlock`` of ``StreamLayer`` with
``SideBySideMixer(WindowAttention, SelectiveScanMixer)`` and ``MoELayer`` (``TopKRouter``, fused dispatcher, ``GroupedMLP``
with ``ClampedGLU``, ``SharedExpertMLP``), a column-parallel output layer.  It follows the ``GPTModel`` call signature, so the
engines, the generation server and the trace replayer drive it like any other language model.
"""
from __future__ import annotations

import torch

from ...moe.experts import GroupedMLP
from ...moe.moe_layer import MoELayer, MoESubmodules
from ...moe.shared_experts import SharedExpertMLP
from ...parallel.tp_layers import ColumnParallelLinear, RowParallelLinear
from ...ssm.selective_scan import SelectiveScanMixer
from ...transformer.hybrid_layer import StreamBlock, StreamLayer
from ...transformer.mlp import MLPSubmodules
from ...transformer.side_by_side import SideBySideMixer
from ...transformer.spec_utils import ModuleSpec
from ...transformer.window_attention import WindowAttention
from ..common.embeddings import LanguageModelEmbedding
from ..common.language_module import LanguageModule
from .config import SLOPE_EXPONENT, DomasunConfig

_MLP_SUB = MLPSubmodules(linear_fc1=ColumnParallelLinear, linear_fc2=RowParallelLinear)


def build_mixer(dcfg: DomasunConfig, base, index: int):
    l = dcfg.layers[index]
    mx = l.mixer
    if l.type == "parallel":
        a, r = mx["left"], mx["right"]
        left = WindowAttention(base, index, int(a["heads"]), int(a.get("kv_heads", a["heads"])), int(a["dim"]),
                               int(a.get("vdim", a["dim"])), float(a["scale"]), int((a.get("mask") or {}).get("size", 0)),
                               sink=True, slope_exponent=SLOPE_EXPONENT, qk_norm=True, values_are_keys=True, head_gate=True,
                               bias=True, eps=dcfg.norm_eps)
        right = SelectiveScanMixer(base, index, int(r["inner"]), int(r["state"]), int(r["dt_rank"]), int(r.get("conv", 1)))
        return SideBySideMixer(base, index, left, right, "scaled_sum", float(mx.get("left_scale", 1.0)),
                               float(mx.get("right_scale", 1.0)))
    raise ValueError(f"unknown mixer type {l.type!r}")


def build_mlp(dcfg: DomasunConfig, base, index: int):
    mlp = dcfg.layers[index].mlp
    if not mlp:
        return None
    sub = MoESubmodules(experts=ModuleSpec(module=GroupedMLP, submodules=_MLP_SUB),
                        shared_experts=ModuleSpec(module=SharedExpertMLP, params={"gate": True}, submodules=_MLP_SUB))
    return MoELayer(dcfg.mlp_transformer_config(base, mlp), sub, layer_number=index)


class DomasunModel(LanguageModule):
    def __init__(self, dcfg: DomasunConfig, config=None, pre_process: bool = True, post_process: bool = True,
                 parallel_output: bool = False, max_sequence_length: int = 0):
        config = config or dcfg.base_transformer_config()
        super().__init__(config)
        self.dcfg = dcfg
        self.vocab_size, self.max_sequence_length = dcfg.vocab, max_sequence_length
        self.pre_process, self.post_process = pre_process, post_process
        self.share_embeddings_and_output_weights = False
        self.model_type = "encoder_or_decoder"
        self.logit_softcap = dcfg.logit_softcap
        if pre_process:
            self.embedding = LanguageModelEmbedding(config, dcfg.vocab, max_sequence_length, "sinusoidal")
        streams, hyper = dcfg.streams or 1, dcfg.streams is not None
        builders = [(lambda i: StreamLayer(config, i, build_mixer(dcfg, config, i), build_mlp(dcfg, config, i), streams,
                                           learned_connections=hyper, layer_scale=True)) for _ in dcfg.layers]
        self.decoder = StreamBlock(config, builders, dcfg.runs(), streams, post_process=post_process)
        if post_process:
            self.output_layer = ColumnParallelLinear(config.hidden_size, dcfg.vocab, config=config, init_method=config.init_method,
                                                     bias=False, skip_bias_add=False, gather_output=not parallel_output)
        self.setup_embeddings_and_output_layer()

    def set_input_tensor(self, t):
        self.decoder.set_input_tensor(t[0] if isinstance(t, (list, tuple)) else t)

    def forward(self, input_ids, position_ids=None, attention_mask=None, decoder_input=None, labels=None,
                inference_context=None, inference_params=None, **_):
        inference_context = inference_context or inference_params
        x = decoder_input
        if x is None and self.pre_process:
            x = self.embedding(input_ids=input_ids, position_ids=position_ids)
        h = self.decoder(x, inference_context=inference_context)
        if not self.post_process:
            return h
        logits, _ = self.output_layer(h)
        if self.logit_softcap:
            logits = self.logit_softcap * torch.tanh(logits.float() / self.logit_softcap)
        if labels is None:
            return logits.transpose(0, 1).contiguous()
        return self.compute_language_model_loss(labels, logits)
