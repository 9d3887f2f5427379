"""Configuration of Domasun models: the ``config.json`` reader and its mapping onto the framework's configs.

``config.json`` keys: ``architecture``, ``vocab``, ``width``, ``norm.eps``, ``streams`` (the number of residual streams of
the hyper-connections; absent: one stream with the plain residual sum), ``logit_softcap`` (absent: none), ``loop``
(``start``, ``stop``, ``times``: layers ``start .. stop - 1`` run ``times`` times in a row with the same weights, each pass
with a cache and state of its own; absent: every layer once) and ``layers``: a list whose entries carry ``type``
(``parallel``), the mixer's sizes under ``mixer`` and the feed-forward under ``mlp`` (``null``: none).

* ``parallel``: ``mixer.left`` = attention (``heads``, ``kv_heads``, ``dim``, ``vdim``, ``scale``, ``mask.size`` = the sliding
  window); ``mixer.right`` = selective scan (``inner``, ``state``, ``dt_rank``, ``conv`` taps); ``left_scale`` and
  ``right_scale`` weigh the two results.
* ``mlp.kind`` ``moe``: ``expert`` (``ff``, ``limit``), ``router`` (``experts``, ``top``) and optionally ``shared``
  (``ff``, ``limit``), a gated expert that every token runs.
"""
from __future__ import annotations

import dataclasses
import json
import os
from dataclasses import dataclass
from typing import Any, Dict, List, Optional

import torch

from ...config.transformer_config import TransformerConfig
from ...transformer.mlp import ClampedGLU

MIXER_TYPES = ("parallel",)
MLP_KINDS = ("moe",)
SLOPE_EXPONENT = 8.0        # head h's distance penalty is 2^(-8 (h + 1) / heads)
GLU_ALPHA, GLU_SHIFT = 1.702, 1.0


@dataclass
class DomasunLayerConfig:
    type: str
    mixer: Dict[str, Any]
    mlp: Optional[Dict[str, Any]] = None


@dataclass
class DomasunConfig:
    vocab: int
    width: int
    layers: List[DomasunLayerConfig]
    norm_eps: float = 1e-5
    streams: Optional[int] = None            # None: no hyper-connections
    logit_softcap: Optional[float] = None
    loop: Optional[Dict[str, int]] = None
    architecture: str = "Domasun"

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "DomasunConfig":
        layers = []
        for i, l in enumerate(d["layers"]):
            if l["type"] not in MIXER_TYPES:
                raise ValueError(f"layer {i}: unknown mixer type {l['type']!r}")
            if l.get("mlp") and l["mlp"].get("kind", "moe") not in MLP_KINDS:
                raise ValueError(f"layer {i}: unknown mlp kind {l['mlp'].get('kind')!r}")
            layers.append(DomasunLayerConfig(l["type"], dict(l["mixer"]), dict(l["mlp"]) if l.get("mlp") else None))
        loop = d.get("loop")
        if loop:
            loop = {k: int(loop[k]) for k in ("start", "stop", "times")}
            if not (0 <= loop["start"] <= loop["stop"] <= len(layers)) or loop["times"] < 1:
                raise ValueError(f"loop {loop} does not fit {len(layers)} layers")
        cap = d.get("logit_softcap")
        return cls(vocab=int(d["vocab"]), width=int(d["width"]), layers=layers,
                   norm_eps=float((d.get("norm") or {}).get("eps", 1e-5)),
                   streams=None if d.get("streams") is None else int(d["streams"]),
                   logit_softcap=float(cap) if cap else None, loop=loop or None,
                   architecture=d.get("architecture", "Domasun"))

    @classmethod
    def from_json(cls, path: str) -> "DomasunConfig":
        if os.path.isdir(path):
            path = os.path.join(path, "config.json")
        with open(path) as f:
            return cls.from_dict(json.load(f))

    def runs(self) -> List[int]:
        """The layer that runs at every depth: the looped span repeated ``times`` times in a row."""
        n = len(self.layers)
        if not self.loop:
            return list(range(n))
        a, b, k = self.loop["start"], self.loop["stop"], self.loop["times"]
        return list(range(a)) + list(range(a, b)) * k + list(range(b, n))

    # -- mapping onto the framework's TransformerConfig ---------------------------------------------------------------------
    def base_transformer_config(self, params_dtype=torch.bfloat16, use_cpu_initialization: Optional[bool] = None,
                                perform_initialization: bool = True, **overrides) -> TransformerConfig:
        cpu = (not torch.cuda.is_available()) if use_cpu_initialization is None else use_cpu_initialization
        kw = dict(num_layers=len(self.layers), hidden_size=self.width, num_attention_heads=1, kv_channels=self.width,
                  ffn_hidden_size=self.width, normalization="LayerNorm", layernorm_epsilon=self.norm_eps, add_bias_linear=False,
                  gated_linear_unit=True, activation_func=ClampedGLU(1.0, GLU_ALPHA, GLU_SHIFT), hidden_dropout=0.0,
                  attention_dropout=0.0, params_dtype=params_dtype, bf16=params_dtype == torch.bfloat16,
                  fp16=params_dtype == torch.float16, fp32_residual_connection=True, use_cpu_initialization=cpu,
                  perform_initialization=perform_initialization, bias_activation_fusion=False)
        kw.update(overrides)
        return TransformerConfig(**kw)

    @staticmethod
    def mlp_transformer_config(base: TransformerConfig, mlp: Dict[str, Any]) -> TransformerConfig:
        """The config a layer's mixture of experts is built from: top-k of the router logits, softmax over the chosen
        ones, clamped gated experts, and the gated shared expert with a clamp of its own."""
        r, ex, shared = mlp["router"], mlp["expert"], mlp.get("shared")
        return dataclasses.replace(
            base, num_moe_experts=int(r["experts"]), moe_router_topk=int(r["top"]), moe_ffn_hidden_size=int(ex["ff"]),
            ffn_hidden_size=int(ex["ff"]), gated_linear_unit=True, activation_func=ClampedGLU(float(ex["limit"]), GLU_ALPHA, GLU_SHIFT),
            moe_router_pre_softmax=False, moe_router_score_function="softmax", moe_router_dtype="fp32",
            moe_router_load_balancing_type="none", moe_aux_loss_coeff=0.0, moe_token_dispatcher_type="fused",
            moe_grouped_gemm=True, moe_shared_expert_intermediate_size=int(shared["ff"]) if shared else None,
            moe_shared_expert_gate=bool(shared),
            moe_shared_expert_activation_func=ClampedGLU(float(shared["limit"]), GLU_ALPHA, GLU_SHIFT) if shared else None)
