"""Zikunex: a decoder-only hybrid whose layers pick their sequence mixer -- latent attention (optionally reading
another layer's cached latents), a gated delta-rule memory with per-channel decay, or an mLSTM matrix memory -- and a
dense or mixture-of-experts squared-ReLU feed-forward, around an fp32 residual stream.

The model is assembled from the framework's parts: ``LanguageModelEmbedding`` (scaled), ``ResidualF32Block`` of
``ResidualF32Layer`` with ``LatentSelfAttention`` / ``GatedDeltaMixer`` / ``MLSTMMixer``, ``MLP`` or ``MoELayer``
(``TopKRouter`` with max-scored group-limited routing, all-gather dispatcher, grouped experts, shared expert), and a
column-parallel output layer.  It follows the ``GPTModel`` call signature (``forward(input_ids, position_ids,
attention_mask, inference_context=...) -> [b, s, V]`` logits or the per-token loss when ``labels`` is given), so the
engines, the generation server and the pipeline helpers drive it like any other language model.
"""
from __future__ import annotations

import dataclasses
from typing import Optional

import torch

from ...moe.experts import GroupedMLP
from ...moe.moe_layer import MoELayer, MoESubmodules
from ...moe.shared_experts import SharedExpertMLP
from ...parallel.tp_layers import ColumnParallelLinear, RowParallelLinear
from ...ssm.gated_delta import GatedDeltaMixer
from ...ssm.mlstm import MLSTMMixer
from ...transformer.hybrid_layer import ResidualF32Block, ResidualF32Layer
from ...transformer.mla import LatentSelfAttention
from ...transformer.mlp import MLP, MLPSubmodules
from ...transformer.spec_utils import ModuleSpec
from ..common.embeddings import LanguageModelEmbedding
from ..common.language_module import LanguageModule
from .config import ZikunexConfig

_MLP_SUB = MLPSubmodules(linear_fc1=ColumnParallelLinear, linear_fc2=RowParallelLinear)
DEFAULT_LOW_RANK = 16


def build_mixer(zcfg: ZikunexConfig, base, index: int):
    l = zcfg.layers[index]
    mx = l.mixer
    if l.type == "latent_attention":
        return LatentSelfAttention(base, index, int(mx["heads"]), int(mx["dim"]), int(mx["vdim"]), int(mx["kv_rank"]),
                                   int(mx["q_rank"]), float(mx["scale"]), mx.get("kv_from"), zcfg.norm_eps)
    if l.type == "channel_delta":
        return GatedDeltaMixer(base, index, int(mx["heads"]), int(mx.get("kv_heads", mx["heads"])), int(mx["dim"]),
                               int(mx["vdim"]), int(mx["conv"]), int(mx.get("decay_rank", DEFAULT_LOW_RANK)),
                               int(mx.get("gate_rank", DEFAULT_LOW_RANK)), zcfg.norm_eps)
    if l.type == "mlstm":
        return MLSTMMixer(base, index, int(mx["heads"]), int(mx["dim"]), int(mx["vdim"]), float(mx["gate_cap"]), zcfg.norm_eps)
    raise ValueError(f"unknown mixer type {l.type!r}")


def build_mlp(zcfg: ZikunexConfig, base, index: int):
    mlp = zcfg.layers[index].mlp
    if not mlp:
        return None
    cfg = zcfg.mlp_transformer_config(base, mlp)
    if mlp["kind"] == "dense":
        return MLP(cfg, _MLP_SUB)
    sub = MoESubmodules(experts=ModuleSpec(module=GroupedMLP, submodules=_MLP_SUB),
                        shared_experts=ModuleSpec(module=SharedExpertMLP, params={"gate": False}, submodules=_MLP_SUB))
    return MoELayer(cfg, sub, layer_number=index)


class ZikunexModel(LanguageModule):
    def __init__(self, zcfg: ZikunexConfig, config=None, pre_process: bool = True, post_process: bool = True,
                 parallel_output: bool = False, max_sequence_length: int = 0):
        config = config or zcfg.base_transformer_config()
        super().__init__(config)
        self.zcfg = zcfg
        self.vocab_size, self.max_sequence_length = zcfg.vocab, max_sequence_length
        self.pre_process, self.post_process = pre_process, post_process
        self.share_embeddings_and_output_weights = False
        self.model_type = "encoder_or_decoder"
        if pre_process:
            self.embedding = LanguageModelEmbedding(config, zcfg.vocab, max_sequence_length, "none")
        self.embedding_scale = float(zcfg.embedding_scale)
        builders = [(lambda i: ResidualF32Layer(config, i, build_mixer(zcfg, config, i), build_mlp(zcfg, config, i)))
                    for _ in zcfg.layers]
        self.decoder = ResidualF32Block(config, builders, post_process=post_process)
        if post_process:
            self.output_layer = ColumnParallelLinear(config.hidden_size, zcfg.vocab, config=config, init_method=config.init_method,
                                                     bias=False, skip_bias_add=False, gather_output=not parallel_output)
        self.setup_embeddings_and_output_layer()

    def set_input_tensor(self, t):
        self.decoder.set_input_tensor(t[0] if isinstance(t, (list, tuple)) else t)

    def forward(self, input_ids, position_ids=None, attention_mask=None, decoder_input=None, labels=None,
                inference_context=None, inference_params=None, **_):
        inference_context = inference_context or inference_params
        x = decoder_input
        if x is None and self.pre_process:
            x = self.embedding(input_ids=input_ids, position_ids=position_ids).float() * self.embedding_scale
        h = self.decoder(x, inference_context=inference_context)
        if not self.post_process:
            return h
        logits, _ = self.output_layer(h)
        if labels is None:
            return logits.transpose(0, 1).contiguous()
        return self.compute_language_model_loss(labels, logits)
