"""Configuration of Nunosun models: the ``config.json`` reader and its mapping onto the framework's configs.

``config.json`` keys: ``architecture``, ``vocab``, ``width``, ``norm.eps``, ``logit_scale`` (absent: 1), ``canon.taps`` (the
causal convolution in front of every mixer; absent or below 2: none), ``token_side.dim`` (the per-layer token vector; absent:
none) and ``layers``: a list whose entries carry ``type`` (``parallel`` or ``delta``), the mixer's sizes under ``mixer`` and
the feed-forward under ``mlp`` (``null``: none).

* ``parallel``: ``mixer.left`` = attention (``heads``, ``kv_heads``, ``dim``, ``vdim``, ``scale``, ``mask.size`` = the sliding
  window, ``bias_max`` = the distance from which the learned bias stays constant); ``mixer.right`` = retention (``heads``,
  ``dim``, ``vdim``, ``decay`` = one number per head, ``rot.dims`` / ``rot.base``).
* ``delta``: gated delta rule (``heads``, ``kv_heads``, ``dim``, ``vdim``, ``conv`` taps).
* ``mlp.kind`` ``dense``: ``ff``; ``moe``: ``expert.ff``, ``router.experts``, ``router.top``.
"""
from __future__ import annotations

import dataclasses
import json
import os
from dataclasses import dataclass
from typing import Any, Dict, List, Optional

import torch
import torch.nn.functional as F

from ...config.transformer_config import TransformerConfig

MIXER_TYPES = ("parallel", "delta")
MLP_KINDS = ("dense", "moe")
UNIT_EPS = 1e-6             # under the root when the delta rule's q and k are made unit vectors


@dataclass
class NunosunLayerConfig:
    type: str
    mixer: Dict[str, Any]
    mlp: Optional[Dict[str, Any]] = None


@dataclass
class NunosunConfig:
    vocab: int
    width: int
    layers: List[NunosunLayerConfig]
    norm_eps: float = 1e-6
    logit_scale: float = 1.0
    canon_taps: int = 0
    side_dim: int = 0
    architecture: str = "Nunosun"

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "NunosunConfig":
        layers = []
        for i, l in enumerate(d["layers"]):
            if l["type"] not in MIXER_TYPES:
                raise ValueError(f"layer {i}: unknown mixer type {l['type']!r}")
            if l.get("mlp") and l["mlp"].get("kind", "dense") not in MLP_KINDS:
                raise ValueError(f"layer {i}: unknown mlp kind {l['mlp'].get('kind')!r}")
            layers.append(NunosunLayerConfig(l["type"], dict(l["mixer"]), dict(l["mlp"]) if l.get("mlp") else None))
        scale = d.get("logit_scale")
        return cls(vocab=int(d["vocab"]), width=int(d["width"]), layers=layers,
                   norm_eps=float((d.get("norm") or {}).get("eps", 1e-6)),
                   logit_scale=1.0 if scale is None else float(scale),
                   canon_taps=int((d.get("canon") or {}).get("taps", 0)),
                   side_dim=int((d.get("token_side") or {}).get("dim", 0)),
                   architecture=d.get("architecture", "Nunosun"))

    @classmethod
    def from_json(cls, path: str) -> "NunosunConfig":
        if os.path.isdir(path):
            path = os.path.join(path, "config.json")
        with open(path) as f:
            return cls.from_dict(json.load(f))

    # -- mapping onto the framework's TransformerConfig ---------------------------------------------------------------------
    def base_transformer_config(self, params_dtype=torch.bfloat16, use_cpu_initialization: Optional[bool] = None,
                                perform_initialization: bool = True, **overrides) -> TransformerConfig:
        cpu = (not torch.cuda.is_available()) if use_cpu_initialization is None else use_cpu_initialization
        kw = dict(num_layers=len(self.layers), hidden_size=self.width, num_attention_heads=1, kv_channels=self.width,
                  ffn_hidden_size=self.width, normalization="RMSNorm", layernorm_epsilon=self.norm_eps, add_bias_linear=False,
                  gated_linear_unit=False, activation_func=F.silu, hidden_dropout=0.0, attention_dropout=0.0,
                  params_dtype=params_dtype, bf16=params_dtype == torch.bfloat16, fp16=params_dtype == torch.float16,
                  fp32_residual_connection=True, use_cpu_initialization=cpu, perform_initialization=perform_initialization,
                  bias_activation_fusion=False)
        kw.update(overrides)
        return TransformerConfig(**kw)

    @staticmethod
    def mlp_transformer_config(base: TransformerConfig, mlp: Dict[str, Any]) -> TransformerConfig:
        """The config a layer's feed-forward is built from.  Dense: one up projection, no gate (the activation is assigned
        by the model).  Mixture of experts: top-k of the biased router logits, softmax over the chosen ones, SiLU-gated
        experts."""
        if mlp.get("kind", "dense") == "dense":
            return dataclasses.replace(base, ffn_hidden_size=int(mlp["ff"]), gated_linear_unit=False)
        r, ex = mlp["router"], mlp["expert"]
        return dataclasses.replace(
            base, num_moe_experts=int(r["experts"]), moe_router_topk=int(r["top"]), moe_ffn_hidden_size=int(ex["ff"]),
            ffn_hidden_size=int(ex["ff"]), gated_linear_unit=True, activation_func=F.silu, moe_router_pre_softmax=False,
            moe_router_score_function="softmax", moe_router_dtype="fp32", moe_router_logit_bias=True,
            moe_router_load_balancing_type="none", moe_aux_loss_coeff=0.0, moe_token_dispatcher_type="fused",
            moe_grouped_gemm=True)
