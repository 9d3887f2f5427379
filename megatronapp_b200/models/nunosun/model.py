"""Nunosun: a decoder-only hybrid.  The word embedding is RMS-normed; every layer has one norm whose output feeds the mixer
(through a short causal convolution over time with a skip) and the feed-forward side by side, their outputs added to the fp32
stream together; after that a per-layer vector of the token, gated by the stream, is projected, normed and added.  Two kinds
of mixer: a gated delta rule with one decay per head, or a sliding-window attention with a learned bias by distance bucket
beside a retention memory with fixed decays and rotary positions, each normed over the width and averaged.  Feed-forwards are
dense with a polynomial-of-norms activation or a mixture of SiLU-gated experts with a biased router.  The logits are scaled.

Assembled from the framework's parts: ``LanguageModelEmbedding`` + ``PerLayerTokenEmbedding``, ``ParallelF32Block`` of
``ParallelF32Layer`` with ``GatedDeltaMixer`` or ``SideBySideMixer(WindowAttention, RetentionMixer)``, ``MLP`` with
``PolyNorm`` or ``MoELayer`` (``TopKRouter``, fused dispatcher, ``GroupedMLP``), ``TokenSideInput``, a column-parallel output
layer.  It follows the ``GPTModel`` call signature, so the engines, the generation server and the trace replayer drive it
like any other language model.
"""
from __future__ import annotations

import torch

from ...moe.experts import GroupedMLP
from ...moe.moe_layer import MoELayer, MoESubmodules
from ...parallel.tp_layers import ColumnParallelLinear, RowParallelLinear
from ...ssm.gated_delta import GatedDeltaMixer
from ...ssm.retention import RetentionMixer
from ...transformer.hybrid_layer import ParallelF32Block, ParallelF32Layer
from ...transformer.mlp import MLP, MLPSubmodules, PolyNorm
from ...transformer.norms import ResidualRMSNorm
from ...transformer.side_by_side import SideBySideMixer
from ...transformer.spec_utils import ModuleSpec
from ...transformer.window_attention import WindowAttention
from ..common.embeddings import LanguageModelEmbedding, PerLayerTokenEmbedding, TokenSideInput
from ..common.language_module import LanguageModule
from .config import UNIT_EPS, NunosunConfig

_MLP_SUB = MLPSubmodules(linear_fc1=ColumnParallelLinear, linear_fc2=RowParallelLinear)


def build_mixer(ncfg: NunosunConfig, base, index: int):
    l = ncfg.layers[index]
    mx = l.mixer
    if l.type == "delta":
        return GatedDeltaMixer(base, index, int(mx["heads"]), int(mx.get("kv_heads", mx["heads"])), int(mx["dim"]),
                               int(mx.get("vdim", mx["dim"])), int(mx.get("conv", 1)), 0, 0, eps=ncfg.norm_eps, unit_eps=UNIT_EPS,
                               decay_per_head=True, gate_act="silu")
    if l.type == "parallel":
        a, r = mx["left"], mx["right"]
        rot = r.get("rot") or {}
        heads = int(a["heads"])
        left = WindowAttention(base, index, heads, int(a.get("kv_heads", heads)), int(a["dim"]), int(a.get("vdim", a["dim"])),
                               float(a["scale"]), int((a.get("mask") or {}).get("size", 0)), sink=False, slope_exponent=None,
                               qk_norm=True, values_are_keys=False, head_gate=False, bias=False, eps=ncfg.norm_eps,
                               bias_buckets=int(a.get("bias_buckets", 0)), bias_max=float(a.get("bias_max", 0.0)))
        right = RetentionMixer(base, index, int(r["heads"]), int(r["dim"]), int(r.get("vdim", r["dim"])), list(r["decay"]),
                               int(rot.get("dims", 0)), float(rot.get("base", 10000.0)), eps=ncfg.norm_eps)
        return SideBySideMixer(base, index, left, right, "normed_mean")
    raise ValueError(f"unknown mixer type {l.type!r}")


def build_mlp(ncfg: NunosunConfig, base, index: int):
    mlp = ncfg.layers[index].mlp
    if not mlp:
        return None
    cfg = ncfg.mlp_transformer_config(base, mlp)
    if mlp.get("kind", "dense") == "dense":
        m = MLP(cfg, _MLP_SUB)
        m.activation_func = PolyNorm(cfg, ncfg.norm_eps)
        return m
    return MoELayer(cfg, MoESubmodules(experts=ModuleSpec(module=GroupedMLP, submodules=_MLP_SUB)), layer_number=index)


class NunosunModel(LanguageModule):
    def __init__(self, ncfg: NunosunConfig, config=None, pre_process: bool = True, post_process: bool = True,
                 parallel_output: bool = False, max_sequence_length: int = 0):
        config = config or ncfg.base_transformer_config()
        super().__init__(config)
        self.ncfg = ncfg
        self.vocab_size, self.max_sequence_length = ncfg.vocab, max_sequence_length
        self.pre_process, self.post_process = pre_process, post_process
        self.share_embeddings_and_output_weights = False
        self.model_type = "encoder_or_decoder"
        self.logit_scale = float(ncfg.logit_scale)
        n = len(ncfg.layers)
        if pre_process:
            self.embedding = LanguageModelEmbedding(config, ncfg.vocab, max_sequence_length, "none")
            self.embedding_norm = ResidualRMSNorm(config, ncfg.width, ncfg.norm_eps, out_dtype=torch.float32)
            self.embedding_norm.weight.data = self.embedding_norm.weight.data.float()      # its output is the fp32 stream
        self.side_embedding = PerLayerTokenEmbedding(config, ncfg.vocab, n, ncfg.side_dim) if ncfg.side_dim else None
        builders = [(lambda i: ParallelF32Layer(config, i, build_mixer(ncfg, config, i), build_mlp(ncfg, config, i), ncfg.canon_taps,
                                                TokenSideInput(config, ncfg.side_dim, ncfg.norm_eps) if ncfg.side_dim else None))
                    for _ in range(n)]
        self.decoder = ParallelF32Block(config, builders, post_process=post_process,
                                        side_slice=self.side_embedding.layer_slice if self.side_embedding is not None else None)
        if post_process:
            self.output_layer = ColumnParallelLinear(config.hidden_size, ncfg.vocab, config=config, init_method=config.init_method,
                                                     bias=False, skip_bias_add=False, gather_output=not parallel_output)
        self.setup_embeddings_and_output_layer()

    def set_input_tensor(self, t):
        self.decoder.set_input_tensor(t[0] if isinstance(t, (list, tuple)) else t)

    def forward(self, input_ids, position_ids=None, attention_mask=None, decoder_input=None, labels=None,
                inference_context=None, inference_params=None, **_):
        inference_context = inference_context or inference_params
        x = decoder_input
        if x is None and self.pre_process:
            x = self.embedding(input_ids=input_ids, position_ids=position_ids).float()
            _, x = self.embedding_norm(x, None)                     # the stream starts as the normed embedding, in fp32
        side = self.side_embedding(input_ids) if self.side_embedding is not None else None
        h = self.decoder(x, inference_context=inference_context, side=side)
        if not self.post_process:
            return h
        logits, _ = self.output_layer(h)
        if self.logit_scale != 1.0:
            logits = logits.float() * self.logit_scale
        if labels is None:
            return logits.transpose(0, 1).contiguous()
        return self.compute_language_model_loss(labels, logits)
