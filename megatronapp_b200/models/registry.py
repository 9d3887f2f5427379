"""Model registry: the architecture name in a model folder's ``config.json`` picks the builder.

A *model folder* holds ``config.json`` (with an ``architecture`` key) and optionally ``model.safetensors``.
``build_model_from_dir`` returns an eval-mode model on ``device`` that follows the ``GPTModel`` call signature, ready for
the inference engines.  New architectures register a builder ``f(path, params_dtype, device, **overrides) -> model``.
"""
from __future__ import annotations

import json
import os
from typing import Callable, Dict

import torch

_BUILDERS: Dict[str, Callable] = {}


def register_architecture(name: str):
    def deco(fn):
        _BUILDERS[name.lower()] = fn
        return fn
    return deco


def architectures():
    return sorted(_BUILDERS)


def architecture_of(path: str) -> str:
    with open(os.path.join(path, "config.json")) as f:
        cfg = json.load(f)
    arch = cfg.get("architecture") or (cfg.get("architectures") or [None])[0]
    if not arch:
        raise ValueError(f"{path}/config.json names no architecture")
    return str(arch)


def build_model_from_dir(path: str, params_dtype=torch.bfloat16, device=None, **overrides):
    arch = architecture_of(path)
    fn = _BUILDERS.get(arch.lower())
    if fn is None:
        raise NotImplementedError(f"architecture {arch!r} is not registered (known: {', '.join(architectures())})")
    return fn(path, params_dtype, device, **overrides)


@register_architecture("Zikunex")
def _zikunex(path, params_dtype, device, **overrides):
    from .zikunex.loader import load_model_dir

    return load_model_dir(path, params_dtype, device, **overrides)


@register_architecture("Lerorax")
def _lerorax(path, params_dtype, device, **overrides):
    from .lerorax.loader import load_model_dir

    return load_model_dir(path, params_dtype, device, **overrides)


@register_architecture("Domasun")
def _domasun(path, params_dtype, device, **overrides):
    from .domasun.loader import load_model_dir

    return load_model_dir(path, params_dtype, device, **overrides)


@register_architecture("Nunosun")
def _nunosun(path, params_dtype, device, **overrides):
    from .nunosun.loader import load_model_dir

    return load_model_dir(path, params_dtype, device, **overrides)


@register_architecture("GPTModel")
def _gpt(path, params_dtype, device, **overrides):
    """A GPT / Llama-style folder: ``config.json`` holds ``TransformerConfig`` fields under ``transformer`` plus
    ``vocab_size``, ``max_sequence_length`` and ``position_embedding_type``; weights (optional) are a safetensors file
    whose names are the model's ``state_dict`` keys."""
    from ..config.transformer_config import TransformerConfig
    from ..parallel import state as ps
    from .gpt.gpt_layer_specs import get_gpt_layer_local_spec
    from .gpt.gpt_model import GPTModel
    from .zikunex.loader import read_safetensors

    if not ps.model_parallel_is_initialized():
        ps.initialize_model_parallel(1, 1)
    with open(os.path.join(path, "config.json")) as f:
        raw = json.load(f)
    kw = dict(raw.get("transformer") or {})
    kw.update(params_dtype=params_dtype, bf16=params_dtype == torch.bfloat16, use_cpu_initialization=True, hidden_dropout=0.0,
              attention_dropout=0.0)
    kw.update(overrides)
    cfg = TransformerConfig(**kw)
    model = GPTModel(cfg, get_gpt_layer_local_spec(cfg.num_moe_experts, cfg.moe_grouped_gemm, normalization=cfg.normalization),
                     int(raw["vocab_size"]), int(raw.get("max_sequence_length", 2048)),
                     position_embedding_type=raw.get("position_embedding_type", "rope"), parallel_output=False)
    st = os.path.join(path, "model.safetensors")
    if os.path.exists(st):
        model.load_state_dict(read_safetensors(st), strict=False)
    if device is not None:
        model = model.to(device)
    return model.eval()
