"""Lerorax: a decoder-only hybrid.  Word embedding plus a hashed bigram embedding; layers that norm their sublayers'
*outputs* (``x <- x + norm(mixer(x))``, ``x <- x + norm(mlp(x))``, zero-centred norm weights, applied as 1 + w) over an fp32 residual
stream; two kinds of mixer -- attention with head mixing side by side with a generalized delta-rule memory, or a minGRU --
and a clamped gated feed-forward.  A layer may run another layer's weights with a cache of its own.

Assembled from the framework's parts: ``LanguageModelEmbedding`` + ``HashedBigramEmbedding``, ``OutputNormF32Block`` of
``OutputNormF32Layer`` with ``SideBySideMixer(MixedHeadAttention, GeneralizedDeltaMixer)`` or ``MinGRUMixer``, ``MLP`` with
``ClampedGLU``, a column-parallel output layer.  It follows the ``GPTModel`` call signature, so the engines, the
generation server and the trace replayer drive it like any other language model.
"""
from __future__ import annotations

import torch

from ...parallel.tp_layers import ColumnParallelLinear, RowParallelLinear
from ...ssm.gen_delta import GeneralizedDeltaMixer
from ...ssm.mingru import MinGRUMixer
from ...transformer.hybrid_layer import OutputNormF32Block, OutputNormF32Layer
from ...transformer.mixed_head_attention import MixedHeadAttention
from ...transformer.mlp import MLP, MLPSubmodules
from ...transformer.side_by_side import SideBySideMixer
from ..common.embeddings import HashedBigramEmbedding, LanguageModelEmbedding
from ..common.language_module import LanguageModule
from .config import DEFAULT_DECAY_RANK, LeroraxConfig

_MLP_SUB = MLPSubmodules(linear_fc1=ColumnParallelLinear, linear_fc2=RowParallelLinear)
NORM_WEIGHT_OFFSET = 1.0          # layer and final norm weights are zero-centred: applied as 1 + w


def build_mixer(lcfg: LeroraxConfig, base, index: int):
    l = lcfg.layers[index]
    mx = l.mixer
    if l.type == "mingru":
        return MinGRUMixer(base, index, int(mx["width"]))
    if l.type == "parallel":
        a, r = mx["left"], mx["right"]
        rot = a.get("rot") or {}
        left = MixedHeadAttention(base, index, int(a["heads"]), int(a.get("kv_heads", a["heads"])), int(a["dim"]),
                                  int(a.get("vdim", a["dim"])), float(a["scale"]), int(a.get("conv", 1)), int(rot.get("dims", 0)),
                                  float(rot.get("base", 10000.0)), rot.get("scaling"), True, lcfg.norm_eps)
        right = GeneralizedDeltaMixer(base, index, int(r["heads"]), int(r["dim"]), int(r.get("vdim", r["dim"])),
                                      int(r.get("decay_rank", DEFAULT_DECAY_RANK)), eps=lcfg.norm_eps)
        return SideBySideMixer(base, index, left, right)
    raise ValueError(f"unknown mixer type {l.type!r}")


def build_mlp(lcfg: LeroraxConfig, base, index: int):
    mlp = lcfg.layers[index].mlp
    return MLP(lcfg.mlp_transformer_config(base, mlp), _MLP_SUB) if mlp else None


class LeroraxModel(LanguageModule):
    def __init__(self, lcfg: LeroraxConfig, config=None, pre_process: bool = True, post_process: bool = True,
                 parallel_output: bool = False, max_sequence_length: int = 0):
        config = config or lcfg.base_transformer_config()
        super().__init__(config)
        self.lcfg = lcfg
        self.vocab_size, self.max_sequence_length = lcfg.vocab, max_sequence_length
        self.pre_process, self.post_process = pre_process, post_process
        self.share_embeddings_and_output_weights = False
        self.model_type = "encoder_or_decoder"
        if pre_process:
            self.embedding = LanguageModelEmbedding(config, lcfg.vocab, max_sequence_length, "none")
            bg = lcfg.bigram
            self.bigram_embedding = HashedBigramEmbedding(config, bg["buckets"], bg["mul_prev"], bg["mul_cur"]) if bg else None
        owners = lcfg.owners()                                      # block layer object p holds the tensors of layer owners[p]
        place = {i: p for p, i in enumerate(owners)}
        builders = [(lambda p, i=i: OutputNormF32Layer(config, i, build_mixer(lcfg, config, i), build_mlp(lcfg, config, i),
                                                      NORM_WEIGHT_OFFSET)) for i in owners]
        self.decoder = OutputNormF32Block(config, builders, [place[lcfg.owner(i)] for i in range(len(lcfg.layers))],
                                          post_process=post_process, weight_offset=NORM_WEIGHT_OFFSET)
        if post_process:
            self.output_layer = ColumnParallelLinear(config.hidden_size, lcfg.vocab, config=config, init_method=config.init_method,
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
            if self.bigram_embedding is not None:
                x = x + self.bigram_embedding(input_ids, inference_context).float()
        h = self.decoder(x, inference_context=inference_context)
        if not self.post_process:
            return h
        logits, _ = self.output_layer(h)
        if labels is None:
            return logits.transpose(0, 1).contiguous()
        return self.compute_language_model_loss(labels, logits)
