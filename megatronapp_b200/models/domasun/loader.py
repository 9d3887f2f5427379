"""Weight loading for Domasun models: the mapping from checkpoint tensor names to the modules' (fused) parameters.

Checkpoint names: ``embed``, ``head``, ``final.norm`` (+ ``.b``), and per layer ``l<i>.norm1``, ``l<i>.norm2`` (+ ``.b``),
``l<i>.ls1``, ``l<i>.ls2``, ``l<i>.hc1.in / .out / .mix``, ``l<i>.hc2.*`` (with hyper-connections), ``l<i>.mix.<name>``,
``l<i>.mlp.<name>``.  Linear weights are stored ``[out, in]`` like the framework's linears, so a mapping is a copy into a
(row slice of a) parameter:

* left: ``left.q, left.k, left.g`` (+ ``.b`` for q / k) are the row segments of the fused ``in_proj`` (the gate's bias rows
  stay zero); ``left.q.norm, left.k.norm, left.o, left.o.b``;
* right: ``right.in, right.conv, right.conv.b, right.x, right.dt, right.dt.b, right.A_log, right.D, right.o``;
* feed-forward: ``router``; ``e<j>.gate`` and ``e<j>.up`` are the halves of expert ``j``'s rows of the grouped ``weight1``,
  ``e<j>.down`` its rows of ``weight2``; ``shared.gate / up / down / sg``.
"""
from __future__ import annotations

import json
import os
from typing import Dict

import torch

from ..zikunex.loader import _copy, read_safetensors


def load_domasun_weights(model, tensors: Dict[str, torch.Tensor], strict: bool = True):
    """Copy checkpoint tensors into ``model`` (a ``DomasunModel`` on a single tensor-parallel rank).  A tensor the model
    needs must be there; tensors the model has no parameter for raise under ``strict`` and are returned otherwise."""
    used = set()

    def take(name):
        if name not in tensors:
            raise KeyError(f"checkpoint has no tensor {name!r}")
        used.add(name)
        return tensors[name]

    def put(param, name, rows=None):
        _copy(param, take(name), name, rows)

    def segments(param, pre, segs, suffix="", only=None):
        o = 0
        for seg, n in segs:
            if only is None or seg in only:
                put(param, f"{pre}{seg}{suffix}", (o, o + n))
            o += n

    def connection(conn, norm, ls, hc):
        put(conn.weight, norm)
        put(conn.bias, norm + ".b")
        put(conn.layer_scale, ls)
        if isinstance(conn.mix, torch.nn.Parameter):
            put(conn.inp, hc + ".in"), put(conn.out, hc + ".out"), put(conn.mix, hc + ".mix")

    put(model.embedding.word_embeddings.weight, "embed")
    put(model.output_layer.weight, "head")
    put(model.decoder.final_layernorm.weight, "final.norm")
    put(model.decoder.final_layernorm.bias, "final.norm.b")
    for i, layer in enumerate(model.decoder.layers):
        connection(layer.mixer_conn, f"l{i}.norm1", f"l{i}.ls1", f"l{i}.hc1")
        a, r, p = layer.mixer.left, layer.mixer.right, f"l{i}.mix."
        segments(a.in_proj.weight, p + "left.", a.segments())
        a.in_proj.bias.data.zero_()
        segments(a.in_proj.bias, p + "left.", a.segments(), ".b", only=("q", "k"))
        for n, prm in (("q.norm", a.q_norm_weight), ("k.norm", a.k_norm_weight), ("o", a.out_proj.weight), ("o.b", a.out_proj.bias)):
            put(prm, p + "left." + n)
        for n, prm in (("in", r.in_proj.weight), ("conv", r.conv_weight), ("conv.b", r.conv_bias), ("x", r.x_proj.weight),
                       ("dt", r.dt_weight), ("dt.b", r.dt_bias), ("A_log", r.A_log), ("D", r.D), ("o", r.out_proj.weight)):
            put(prm, p + "right." + n)
        mlp, m = layer.mlp, f"l{i}.mlp."
        if mlp is None:
            continue
        connection(layer.mlp_conn, f"l{i}.norm2", f"l{i}.ls2", f"l{i}.hc2")
        put(mlp.router.weight, m + "router")
        ex, h = mlp.experts, model.config.hidden_size
        for e in range(ex.num_local_experts):
            put(ex.weight1, f"{m}e{e}.gate", (e * ex.fc1_out, e * ex.fc1_out + ex.ffn))
            put(ex.weight1, f"{m}e{e}.up", (e * ex.fc1_out + ex.ffn, (e + 1) * ex.fc1_out))
            put(ex.weight2, f"{m}e{e}.down", (e * h, (e + 1) * h))
        sh = mlp.shared_experts
        if sh is not None:
            ff = sh.linear_fc2.weight.shape[1]
            put(sh.linear_fc1.weight, m + "shared.gate", (0, ff))
            put(sh.linear_fc1.weight, m + "shared.up", (ff, 2 * ff))
            put(sh.linear_fc2.weight, m + "shared.down")
            put(sh.gate_weight, m + "shared.sg")
    extra = sorted(set(tensors) - used)
    if extra and strict:
        raise ValueError(f"checkpoint tensors without a parameter: {extra[:8]}{' ...' if len(extra) > 8 else ''}")
    return extra


def load_model_dir(path: str, params_dtype=torch.bfloat16, device=None, **config_overrides):
    """Build a ``DomasunModel`` from a folder with ``config.json`` (+ ``model.safetensors``: without it the weights stay
    at their random initialisation) and move it to ``device``."""
    from ...parallel import state as ps
    from .config import DomasunConfig
    from .model import DomasunModel

    if not ps.model_parallel_is_initialized():
        ps.initialize_model_parallel(1, 1)
    with open(os.path.join(path, "config.json")) as f:
        raw = json.load(f)
    st = os.path.join(path, "model.safetensors")
    tensors = read_safetensors(st) if os.path.exists(st) else None
    dcfg = DomasunConfig.from_dict(raw)
    base = dcfg.base_transformer_config(params_dtype, use_cpu_initialization=True, perform_initialization=tensors is None,
                                        **config_overrides)
    model = DomasunModel(dcfg, base)
    if tensors is not None:
        extra = load_domasun_weights(model, tensors, strict=False)
        if extra:
            import sys

            print(f"[domasun] {len(extra)} checkpoint tensors have no parameter and were ignored: {extra[:4]}", file=sys.stderr)
    if device is not None:
        model = model.to(device)
    return model.eval()
