"""Weight loading for Nunosun models: the mapping from checkpoint tensor names to the modules' (fused) parameters.

Checkpoint names: ``embed``, ``embed.norm``, ``side.embed``, ``head``, ``final.norm``, and per layer ``l<i>.norm1``,
``l<i>.canon1``, ``l<i>.side.gate / .proj / .norm``, ``l<i>.mix.<name>``, ``l<i>.mlp.<name>``.  Linear weights are stored
``[out, in]`` like the framework's linears, so a mapping is a copy into a (row slice of a) parameter:

* delta: ``q, k, v, a, g, b`` are the row segments of the fused ``in_proj``; ``q.conv, k.conv, v.conv`` those of the
  convolution; ``A_log, dt_bias, norm, o``;
* parallel, left: ``left.q, left.k, left.v`` are the segments of ``in_proj``; ``left.q.norm, left.k.norm, left.rel, left.o``;
  right: ``right.q, right.k, right.v, right.g`` are the segments of ``in_proj``; ``right.o``; ``left.out`` / ``right.out`` are
  the weights of the two output norms;
* feed-forward: ``up, down, act`` (dense); ``router, router.b``, ``e<j>.gate`` and ``e<j>.up`` are the halves of expert
  ``j``'s rows of the grouped ``weight1``, ``e<j>.down`` its rows of ``weight2``.

Sizes that ``config.json`` leaves to the tensor shapes (the number of distance buckets of the attention bias, omitted
convolution taps) are read from the file's header.
"""
from __future__ import annotations

import json
import os
from typing import Dict

import torch

from ..zikunex.loader import _copy, read_safetensors

DEFAULT_BIAS_BUCKETS = 16           # for a folder without weights whose config does not say


def shapes_into_config(config: dict, shapes: Dict[str, tuple]) -> dict:
    """Fill the sizes that only the tensors carry into the mixer dicts."""
    for i, l in enumerate(config["layers"]):
        mx = l["mixer"]
        if l["type"] == "parallel":
            rel = shapes.get(f"l{i}.mix.left.rel")
            if rel is not None:
                mx["left"]["bias_buckets"] = int(rel[0])
            elif "bias_max" in mx["left"]:
                mx["left"].setdefault("bias_buckets", DEFAULT_BIAS_BUCKETS)
        elif l["type"] == "delta" and "conv" not in mx and f"l{i}.mix.q.conv" in shapes:
            mx["conv"] = int(shapes[f"l{i}.mix.q.conv"][1])
    canon = shapes.get("l0.canon1")
    if canon is not None and not (config.get("canon") or {}).get("taps"):
        config["canon"] = {"taps": int(canon[1])}
    return config


def load_nunosun_weights(model, tensors: Dict[str, torch.Tensor], strict: bool = True):
    """Copy checkpoint tensors into ``model`` (a ``NunosunModel`` on a single tensor-parallel rank).  A tensor the model
    needs must be there; tensors the model has no parameter for raise under ``strict`` and are returned otherwise."""
    used = set()

    def take(name):
        if name not in tensors:
            raise KeyError(f"checkpoint has no tensor {name!r}")
        used.add(name)
        return tensors[name]

    def put(param, name, rows=None):
        _copy(param, take(name), name, rows)

    def segments(param, pre, segs, suffix="", names=None):
        o = 0
        for seg, n in segs:
            put(param, f"{pre}{(names or {}).get(seg, seg)}{suffix}", (o, o + n))
            o += n

    put(model.embedding.word_embeddings.weight, "embed")
    put(model.embedding_norm.weight, "embed.norm")
    if model.side_embedding is not None:
        put(model.side_embedding.weight, "side.embed")
    put(model.output_layer.weight, "head")
    put(model.decoder.final_layernorm.weight, "final.norm")
    for i, layer in enumerate(model.decoder.layers):
        put(layer.input_layernorm.weight, f"l{i}.norm1")
        if layer.taps > 1:
            put(layer.input_conv_weight, f"l{i}.canon1")
        if layer.token_side is not None:
            ts = layer.token_side
            put(ts.gate.weight, f"l{i}.side.gate"), put(ts.proj.weight, f"l{i}.side.proj"), put(ts.norm_weight, f"l{i}.side.norm")
        p, kind = f"l{i}.mix.", model.ncfg.layers[i].type
        if kind == "delta":
            mx = layer.mixer
            segments(mx.in_proj.weight, p, mx.segments(), names={"a1": "a", "g1": "g"})
            segments(mx.conv_weight, p, mx.segments()[:3], ".conv")
            for n, prm in (("A_log", mx.A_log), ("dt_bias", mx.dt_bias), ("norm", mx.norm_weight), ("o", mx.out_proj.weight)):
                put(prm, p + n)
        else:
            a, r = layer.mixer.left, layer.mixer.right
            segments(a.in_proj.weight, p + "left.", a.segments())
            for n, prm in (("q.norm", a.q_norm_weight), ("k.norm", a.k_norm_weight), ("o", a.out_proj.weight)):
                put(prm, p + "left." + n)
            if a.bias_buckets:
                put(a.rel_bias, p + "left.rel")
            segments(r.in_proj.weight, p + "right.", r.segments())
            put(r.out_proj.weight, p + "right.o")
            put(layer.mixer.left_out_weight, p + "left.out")
            put(layer.mixer.right_out_weight, p + "right.out")
        mlp, m = layer.mlp, f"l{i}.mlp."
        if mlp is None:
            continue
        if model.ncfg.layers[i].mlp.get("kind", "dense") == "dense":
            put(mlp.linear_fc1.weight, m + "up"), put(mlp.linear_fc2.weight, m + "down"), put(mlp.activation_func.coef, m + "act")
            continue
        put(mlp.router.weight, m + "router")
        put(mlp.router.logit_bias, m + "router.b")
        ex, h = mlp.experts, model.config.hidden_size
        for e in range(ex.num_local_experts):
            put(ex.weight1, f"{m}e{e}.gate", (e * ex.fc1_out, e * ex.fc1_out + ex.ffn))
            put(ex.weight1, f"{m}e{e}.up", (e * ex.fc1_out + ex.ffn, (e + 1) * ex.fc1_out))
            put(ex.weight2, f"{m}e{e}.down", (e * h, (e + 1) * h))
    extra = sorted(set(tensors) - used)
    if extra and strict:
        raise ValueError(f"checkpoint tensors without a parameter: {extra[:8]}{' ...' if len(extra) > 8 else ''}")
    return extra


def load_model_dir(path: str, params_dtype=torch.bfloat16, device=None, **config_overrides):
    """Build a ``NunosunModel`` from a folder with ``config.json`` (+ ``model.safetensors``: without it the weights stay
    at their random initialisation) and move it to ``device``."""
    from ...parallel import state as ps
    from .config import NunosunConfig
    from .model import NunosunModel

    if not ps.model_parallel_is_initialized():
        ps.initialize_model_parallel(1, 1)
    with open(os.path.join(path, "config.json")) as f:
        raw = json.load(f)
    st = os.path.join(path, "model.safetensors")
    tensors = read_safetensors(st) if os.path.exists(st) else None
    raw = shapes_into_config(raw, {k: tuple(v.shape) for k, v in tensors.items()} if tensors is not None else {})
    ncfg = NunosunConfig.from_dict(raw)
    base = ncfg.base_transformer_config(params_dtype, use_cpu_initialization=True, perform_initialization=tensors is None,
                                        **config_overrides)
    model = NunosunModel(ncfg, base)
    if tensors is not None:
        extra = load_nunosun_weights(model, tensors, strict=False)
        if extra:
            import sys

            print(f"[nunosun] {len(extra)} checkpoint tensors have no parameter and were ignored: {extra[:4]}", file=sys.stderr)
    if device is not None:
        model = model.to(device)
    return model.eval()
