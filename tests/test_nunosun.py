"""Nunosun models in the framework against a plain, slow evaluation of the design's equations (``nunosun_oracle``).

Each test builds its own small configuration and random (or hand-made) weights, loads them through the product loader
and drives the model through the dynamic engine -- whole prompts, prompts cut into portions, token-by-token decoding,
mixed batches, reused pages and state rows -- on the CPU (PyTorch op path) and, marked ``gpu``, on the sm_100a kernels.
"""
import copy
import json
import os
import struct
import subprocess
import sys

import pytest
import torch

import nunosun_oracle as oracle
from megatronapp_b200.data.tokenizer import NullTokenizer
from megatronapp_b200.inference import DynamicInferenceEngine, SamplingParams
from megatronapp_b200.inference.trace import TraceReplayer
from megatronapp_b200.models.nunosun import NunosunConfig, NunosunModel
from megatronapp_b200.models.nunosun.loader import load_nunosun_weights, shapes_into_config
from megatronapp_b200.ops import seqmix
from megatronapp_b200.parallel import state as ps
from megatronapp_b200.transformer.mixed_head_attention import dense_pages
from megatronapp_b200.transformer.window_attention import distance_buckets

DEVICES = ["cpu", pytest.param("cuda", marks=pytest.mark.gpu)]
VOCAB = 61

LEFT = {"heads": 4, "kv_heads": 2, "dim": 8, "vdim": 12, "scale": 0.35, "mask": {"size": 9}, "bias_max": 30}
LEFT_B = {"heads": 3, "kv_heads": 3, "dim": 20, "vdim": 20, "scale": 0.2, "mask": {"size": 5}, "bias_max": 12}
LEFT_C = {"heads": 6, "kv_heads": 1, "dim": 16, "vdim": 8, "scale": 0.25, "mask": {"size": 64}, "bias_max": 40}
RIGHT = {"heads": 3, "dim": 8, "vdim": 12, "decay": [0.9, 0.97, 0.995], "rot": {"dims": 8, "base": 50.0}}
RIGHT_B = {"heads": 2, "dim": 20, "vdim": 10, "decay": [0.8, 0.99], "rot": {"dims": 6, "base": 10000.0}}       # part of a head turns
RIGHT_C = {"heads": 5, "dim": 12, "vdim": 36, "decay": [0.5, 0.9, 0.95, 0.99, 0.999], "rot": {"dims": 0, "base": 1.0}}   # none does
PAR = {"type": "parallel", "mixer": {"left": LEFT, "right": RIGHT}}
PAR_B = {"type": "parallel", "mixer": {"left": LEFT_B, "right": RIGHT_B}}
PAR_C = {"type": "parallel", "mixer": {"left": LEFT_C, "right": RIGHT_C}}
DELTA = {"type": "delta", "mixer": {"heads": 4, "kv_heads": 2, "dim": 8, "vdim": 12, "conv": 3}}
DELTA_B = {"type": "delta", "mixer": {"heads": 3, "kv_heads": 3, "dim": 20, "vdim": 6, "conv": 2}}
DELTA_C = {"type": "delta", "mixer": {"heads": 6, "kv_heads": 1, "dim": 36, "vdim": 40, "conv": 5}}
DENSE = {"kind": "dense", "ff": 48}
DENSE_B = {"kind": "dense", "ff": 20}
MOE = {"kind": "moe", "expert": {"ff": 16}, "router": {"experts": 5, "top": 2}}
MOE_B = {"kind": "moe", "expert": {"ff": 8}, "router": {"experts": 3, "top": 1}}
MOE_C = {"kind": "moe", "expert": {"ff": 24}, "router": {"experts": 4, "top": 4}}


def layer(spec, mlp=None):
    l = copy.deepcopy(spec)
    l["mlp"] = copy.deepcopy(mlp)
    return l


def config_of(layers, width=32, vocab=VOCAB, eps=1e-5, taps=3, side=6, logit_scale=0.5):
    cfg = {"architecture": "Nunosun", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}
    if taps is not None:
        cfg["canon"] = {"taps": taps}
    if side is not None:
        cfg["token_side"] = {"dim": side}
    if logit_scale is not None:
        cfg["logit_scale"] = logit_scale
    return cfg


HYBRID = config_of([layer(DELTA, DENSE), layer(PAR, MOE), layer(PAR_B, DENSE_B), layer(DELTA_B, MOE_B), layer(PAR_C)])


def build(cfg, device, dtype=torch.float32, seed=0, weights=None):
    if not ps.model_parallel_is_initialized():
        ps.initialize_model_parallel(1, 1)
    W = weights if weights is not None else oracle.random_weights(cfg, seed)
    raw = shapes_into_config(copy.deepcopy(cfg), {k: tuple(v.shape) for k, v in W.items()})
    ncfg = NunosunConfig.from_dict(raw)
    model = NunosunModel(ncfg, ncfg.base_transformer_config(dtype, use_cpu_initialization=True, perform_initialization=False))
    load_nunosun_weights(model, W)
    return model.to(device).eval(), W


def replayer(model, max_tokens=512, block_size=4, max_requests=4):
    return TraceReplayer(model, max_tokens, block_size=block_size, max_requests=max_requests, max_sequence_length=4096)


def run_cut(rp, rid, tokens, cuts):
    """Feed ``tokens`` in portions of the given sizes (the rest one by one); logits of every position."""
    outs, at = [], 0
    sizes = list(cuts)
    while at < len(tokens):
        n = sizes.pop(0) if sizes else 1
        n = min(n, len(tokens) - at)
        outs.append(rp.step([{"id": rid, "tokens": tokens[at:at + n], "want": list(range(n))}]))
        at += n
    rp.step([], end=[rid])
    return torch.cat(outs)


def tokens_of(n, vocab=VOCAB, seed=0):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


def close(got, want, tol):
    want = want.to(torch.float64)
    err = (got.to(torch.float64).cpu() - want).abs().max().item()
    assert err <= tol * max(1.0, want.abs().max().item()), f"max error {err:.3e} (scale {want.abs().max().item():.3e})"


TOL = {torch.float32: 2e-4, torch.bfloat16: 6e-2}


def close_in_16_bits(got, want, typical=3e-2, outlier=0.15, share=0.1):
    """Rounding to 16 bits is amplified where a norm divides by something small, so a few positions may be far off; the typical
    position must be near: the error per position (root mean square over the vocabulary, relative to the logits' scale)."""
    want = want.to(torch.float64)
    rel = (got.to(torch.float64).cpu() - want).pow(2).mean(-1).sqrt() / want.pow(2).mean().sqrt()
    assert float(rel.median()) <= typical and float((rel > outlier).double().mean()) <= share, \
        f"median {float(rel.median()):.3e}, worst {float(rel.max()):.3e}"


def only_branch(W, layer_index, keep):
    """Silence one branch of a parallel mixer: the weight of its output norm becomes zero."""
    W = dict(W)
    gone = "right" if keep == "left" else "left"
    W[f"l{layer_index}.mix.{gone}.out"] = torch.zeros_like(W[f"l{layer_index}.mix.{gone}.out"])
    return W


# ---------------------------------------------------------------------------------------------------------------------
# every mechanism alone: one layer, whole prompt and cut prompt
# ---------------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("spec,keep,kw", [
    (layer(PAR), "left", dict(taps=None, side=None)), (layer(PAR), "right", dict(taps=None, side=None)), (layer(PAR_B), None, dict(side=None)),
    (layer(PAR_C), None, dict(taps=None)), (layer(DELTA), None, dict(taps=None, side=None, logit_scale=None)), (layer(DELTA_C), None, dict(taps=4)),
    (layer(DELTA_B, DENSE), None, dict(taps=2, side=None)), (layer(DELTA, MOE), None, dict(side=3)), (layer(DELTA, MOE_B), None, dict(taps=None)),
    (layer(PAR, MOE_C), None, dict())],
    ids=["attention", "retention", "parallel_conv", "parallel_side", "delta", "delta_wide_conv4", "dense_polynorm", "moe", "moe_top1",
         "moe_all_experts"])
def test_single_mechanism_matches_oracle(spec, keep, kw, device):
    cfg = config_of([spec], **kw)
    W = oracle.random_weights(cfg, 1)
    if keep:
        W = only_branch(W, 0, keep)
    model, W = build(cfg, device, weights=W)
    toks = tokens_of(37)
    want, layers = oracle.forward(cfg, W, toks, return_layers=True)
    seen = []
    model.decoder.tap = lambda i, x: seen.append(x.detach().float().cpu().clone())
    rp = replayer(model)
    close(run_cut(rp, "a", toks, [len(toks)]), want, TOL[torch.float32])
    close(seen[0].view(len(toks), -1), layers[0], TOL[torch.float32])
    model.decoder.tap = None
    close(run_cut(rp, "b", toks, [17, 2, 16]), want, TOL[torch.float32])


def test_whole_sequence_forward_without_a_context():
    """The training-style call (``[b, s]`` ids, no inference context) runs the same mixers from zero state."""
    for cfg in (HYBRID, config_of([layer(PAR_B, MOE), layer(DELTA_B)], side=None, logit_scale=None)):
        model, W = build(cfg, "cpu")
        a, b = tokens_of(21, seed=1), tokens_of(21, seed=2)
        out = model(torch.tensor([a, b]), None, None)
        close(out[0], oracle.forward(cfg, W, a), TOL[torch.float32])
        close(out[1], oracle.forward(cfg, W, b), TOL[torch.float32])


@pytest.mark.parametrize("device", DEVICES)
def test_ops_match_the_oracle_functions(device):
    """The op level: attention with the bucketed bias, retention with rotation, the per-head delta rule, residual convolution,
    PolyNorm, the GELU gate, the head norm with a SiLU gate and the additions -- each against the oracle's function."""
    g = torch.Generator().manual_seed(3)
    rnd = lambda *s: torch.randn(*s, generator=g)  # noqa: E731
    d = lambda t: t.to(device)  # noqa: E731
    T = 9
    # attention: two sequences of 9 tokens, H = 4 over G = 2, values wider than keys, 6 buckets up to distance 7
    H, G, dd, dv, B, D = 4, 2, 6, 10, 6, 7.0
    q, k, v, rel = rnd(2 * T, H, dd), rnd(2 * T, G, dd), rnd(2 * T, G, dv), rnd(B, H)
    table, tok_req, tok_len = dense_pages(T, 2, device)
    for window in (4, 0, 9):
        length = min(window, 9) if window else 9
        bias = rel[distance_buckets(B, D, length)]
        got = seqmix.window_attention_paged(d(q), d(k), d(v), table, tok_req, tok_len, T, 0.4, window, dist_bias=d(bias))
        for r in range(2):
            sl = slice(r * T, (r + 1) * T)
            want = oracle.window_attention(q[sl].double(), k[sl].double(), v[sl].double(), 0.4, window, rel.double(), D)
            close(got[sl].view(T, H, dv), want, 1e-5)
    # retention: three sequences with carried memory, part of the head turns
    Hr, dr, dvr, rot = 3, 10, 7, 6
    lens = [5, 1, 9]
    qs, ks, vs = rnd(sum(lens), Hr, dr), rnd(sum(lens), Hr, dr), rnd(sum(lens), Hr, dvr)
    decay = torch.tensor([0.7, 0.95, 1.0])
    cu = [0, 5, 6, 15]
    pos = torch.cat([torch.arange(n) for n in lens])
    state = torch.zeros(4, Hr, dr, dvr, device=device)
    got = seqmix.retention_scan(d(qs), d(ks), d(vs), d(decay), seqmix.PackedBatch(cu, [3, 0, 1], device), state, d(pos),
                                d(seqmix.rotary_frequencies(rot, 100.0)), dr ** -0.5)
    for r in range(3):
        sl = slice(cu[r], cu[r + 1])
        p = list(range(lens[r]))
        want = oracle.retention(oracle.rotate_half(qs[sl].double(), p, rot, 100.0), oracle.rotate_half(ks[sl].double(), p, rot, 100.0) * dr ** -0.5,
                                vs[sl].double(), decay.double())
        close(got[sl], want, 1e-5)
    assert float(state[2].abs().max()) == 0.0                       # a row no sequence of the step owns stays untouched
    # wide keys and sequences longer than a staging round (the prompt instances of the kernel), fed in two steps
    for dk, dvv, nrot in ((64, 40, 32), (128, 24, 8), (72, 130, 0)):
        n, cut = 45, 20
        qw, kw, vw = rnd(n, 2, dk), rnd(n, 2, dk), rnd(n, 2, dvv)
        dec = torch.tensor([0.9, 0.99])
        inv = seqmix.rotary_frequencies(2 * nrot, 1000.0)
        st = torch.zeros(1, 2, dk, dvv, device=device)
        got = torch.cat([seqmix.retention_scan(d(qw[lo:hi]), d(kw[lo:hi]), d(vw[lo:hi]), d(dec), seqmix.PackedBatch([0, hi - lo], [0], device), st,
                                               d(torch.arange(lo, hi)), None if inv is None else d(inv), dk ** -0.5) for lo, hi in ((0, cut), (cut, n))])
        p = list(range(n))
        want = oracle.retention(oracle.rotate_half(qw.double(), p, 2 * nrot, 1000.0), oracle.rotate_half(kw.double(), p, 2 * nrot, 1000.0) * dk ** -0.5,
                                vw.double(), dec.double())
        close(got, want, 1e-5)
    # delta rule with one decay per head, grouped q / k heads
    Hd, Gd = 4, 2
    qd, kd, vd = rnd(T, Gd, dd), rnd(T, Gd, dd), rnd(T, Hd, dv)
    gd, bd = torch.rand(T, Hd, generator=g) * 0.5 + 0.5, torch.rand(T, Hd, generator=g)
    state = torch.zeros(1, Hd, dd, dv, device=device)
    got = seqmix.delta_rule_scan(d(qd), d(kd), d(vd), d(torch.log(gd)), d(bd), seqmix.PackedBatch([0, T], [0], device), state, 1e-6, dd ** -0.5)
    want = oracle.delta_rule((oracle.unit(qd.double()) * dd ** -0.5).repeat_interleave(2, 1), oracle.unit(kd.double()).repeat_interleave(2, 1),
                             vd.double(), gd.double(), bd.double())
    close(got, want, 1e-5)
    # the delta rule's gates from a strided projection, one decay per head and one per key channel
    proj, A_log = rnd(T, 40), rnd(Hd) * 0.5
    for C in (Hd, Hd * 3):
        dtb = rnd(C)
        ld_, bt_ = seqmix.decay_gates(d(proj)[:, 2:2 + C], d(proj)[:, 20:20 + Hd], d(A_log), d(dtb))
        want_ld = -torch.exp(A_log.double()).repeat_interleave(C // Hd) * oracle.softplus(proj[:, 2:2 + C].double() + dtb.double())
        close(ld_, want_ld, 1e-5), close(bt_, 1.0 / (1.0 + torch.exp(-proj[:, 20:20 + Hd].double())), 1e-5)
    # convolution with the input added, carried over two steps
    C, taps = 10, 3
    u, cw = rnd(T, C), rnd(C, taps)
    win = torch.zeros(1, taps - 1, C, device=device)
    got = torch.cat([seqmix.causal_conv(d(u[:4]), d(cw), seqmix.PackedBatch([0, 4], [0], device), win, residual=True),
                     seqmix.causal_conv(d(u[4:]), d(cw), seqmix.PackedBatch([0, T - 4], [0], device), win, residual=True)])
    close(got, u.double() + oracle.causal_conv(u.double(), cw.double()), 1e-5)
    # PolyNorm on rows of a strided view, the GELU gate times a column slice
    z, coef = rnd(T, 50), torch.tensor([0.7, -0.4, 0.3, 0.2])
    close(seqmix.poly_norm(d(z)[:, 4:44], d(coef), 1e-5), oracle.poly_norm(z[:, 4:44].double(), coef.double(), 1e-5), 1e-5)
    gt, e = rnd(T, 6), rnd(T, 30)
    close(seqmix.gelu_mul(d(gt), d(e)[:, 12:18]), oracle.gelu_tanh(gt.double()) * e[:, 12:18].double(), 1e-5)
    # read-out norm per head without a weight, SiLU gate from a strided view
    o, gate = rnd(T, 3, 8), rnd(T, 40)
    got = seqmix.gated_head_rms_norm(d(o), None, d(gate)[:, 5:29], 1e-5, torch.float32, "silu")
    close(got, oracle.rms(o.double(), 1e-5).reshape(T, 24) * oracle.silu(gate[:, 5:29].double()), 1e-5)
    # the layer's additions: two normed branches + feed-forward, no outer norm; then a normed addend and the next norm
    Wd = 20
    x, a, b, f, wa, wb, ws, wn = rnd(T, Wd), rnd(T, Wd), rnd(T, Wd), rnd(T, Wd), rnd(Wd), rnd(Wd), rnd(Wd), rnd(Wd)
    x1 = x.double() + 0.5 * (oracle.rms(a.double(), 1e-5) * wa.double() + oracle.rms(b.double(), 1e-5) * wb.double()) + f.double()
    gx, gy = seqmix.norm_add(d(x.clone()), d(a), None, 1e-5, torch.float32, 0.0, d(b), d(wa), d(wb), extra=d(f))
    close(gx, x1, 1e-5), close(gy, x1, 1e-5)
    x2 = x.double() + oracle.rms(a.double(), 1e-5) * ws.double()
    gx, gy = seqmix.norm_add(d(x.clone()), d(a), d(ws), 1e-5, torch.float32, next_weight=d(wn))
    close(gx, x2, 1e-5), close(gy, oracle.rms(x2, 1e-5) * wn.double(), 1e-5)
    gx, gy = seqmix.norm_add(d(x.clone()), d(a), None, 1e-5, torch.float32, next_weight=d(wn))
    close(gx, x.double() + a.double(), 1e-5), close(gy, oracle.rms(x.double() + a.double(), 1e-5) * wn.double(), 1e-5)


def test_distance_buckets_follow_the_rule_at_every_edge():
    for B, D in ((32, 128.0), (10, 30.0), (6, 7.0), (8, 1000.0), (4, 2.5)):
        got = distance_buckets(B, D, 1200).tolist()
        assert got == [oracle.bucket(n, B, D) for n in range(1200)]
        assert got[:B // 2] == list(range(B // 2)) and got[B // 2] == B // 2 and max(got) == B - 1


# ---------------------------------------------------------------------------------------------------------------------
# schedules: portions, decoding, batches, reuse
# ---------------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("cuts", [[50], [1], [2, 2, 2], [10, 11, 12], [11, 11], [4, 5, 64 - 9], [33, 3], [47]], ids=str)
def test_portions_and_decoding_match_whole_prompt(cuts, device):
    model, W = build(HYBRID, device)
    toks = tokens_of(50, seed=4)
    want = oracle.forward(HYBRID, W, toks)
    close(run_cut(replayer(model), "a", toks, cuts), want, TOL[torch.float32])


@pytest.mark.parametrize("device", DEVICES)
def test_unequal_batch_matches_each_alone_and_rows_are_reused(device):
    model, W = build(HYBRID, device)
    rp = replayer(model, max_tokens=256, block_size=4, max_requests=3)
    prompts = {"a": tokens_of(23, seed=5), "b": tokens_of(1, seed=6), "c": tokens_of(14, seed=7)}
    want = {k: oracle.forward(HYBRID, W, v) for k, v in prompts.items()}
    cut = {"a": 17, "b": 1, "c": 9}
    out = rp.step([{"id": k, "tokens": v[:cut[k]], "want": list(range(cut[k]))} for k, v in prompts.items()])
    got = {k: [] for k in prompts}
    at = 0
    for k in prompts:
        got[k].append(out[at:at + cut[k]])
        at += cut[k]
    fed = dict(cut)
    live = [k for k in prompts if fed[k] < len(prompts[k])]
    rp.step([], end=[k for k in prompts if k not in live])
    while live:
        out = rp.step([{"id": k, "tokens": prompts[k][fed[k]:fed[k] + 1], "want": [0]} for k in live])
        for n, k in enumerate(live):
            got[k].append(out[n:n + 1])
            fed[k] += 1
        done = [k for k in live if fed[k] == len(prompts[k])]
        live = [k for k in live if k not in done]
        rp.step([], end=done)
    for k in prompts:
        close(torch.cat(got[k]), want[k], TOL[torch.float32])
    # the rows and pages given back are used again by new requests: nothing of the old state may leak
    for n in range(4):
        toks = tokens_of(19 + n, seed=20 + n)
        close(run_cut(rp, f"again{n}", toks, [7, 2]), oracle.forward(HYBRID, W, toks), TOL[torch.float32])


@pytest.mark.parametrize("device", DEVICES)
def test_other_sizes_and_values_that_are_often_equal_or_one(device):
    """One head, one kv head, one expert, one tap (no convolution), two taps, a window of one and one longer than the prompt, no
    rotation and a head that turns whole, a bias table of two rows, decays of one, different heads left and right, no side input,
    layers without feed-forward, another eps, a logit scale of one."""
    left = {"heads": 1, "kv_heads": 1, "dim": 12, "vdim": 12, "scale": 1.0, "mask": {"size": 1}, "bias_max": 4, "bias_buckets": 2}
    right = {"heads": 1, "dim": 4, "vdim": 4, "decay": [1.0], "rot": {"dims": 4, "base": 2.0}}
    one = {"type": "parallel", "mixer": {"left": left, "right": right}}
    d1 = {"type": "delta", "mixer": {"heads": 1, "kv_heads": 1, "dim": 4, "vdim": 4, "conv": 1}}
    moe1 = {"kind": "moe", "expert": {"ff": 4}, "router": {"experts": 1, "top": 1}}
    for cfg in (config_of([layer(one, moe1), layer(PAR_C, MOE), layer(d1)], width=24, taps=1, side=1),
                config_of([layer(DELTA_C, MOE_B), layer(one)], width=40, taps=2, side=None, logit_scale=1.0),
                config_of([layer(PAR_C, MOE_C), layer(d1, DENSE_B)], width=16, eps=1e-3, taps=5, side=9),
                config_of([layer(DELTA_B), layer(PAR_B), layer(DELTA)], width=20, taps=None, logit_scale=None)):
        W = oracle.random_weights(cfg, 11, bias_buckets=7)
        model, W = build(cfg, device, weights=W)
        toks = tokens_of(29, seed=8)
        close(run_cut(replayer(model), "a", toks, [13, 2, 9]), oracle.forward(cfg, W, toks), TOL[torch.float32])


@pytest.mark.parametrize("device", DEVICES)
def test_long_decoding_passes_the_window_over_decoded_tokens(device):
    cfg = config_of([layer(PAR, MOE), layer(DELTA, DENSE_B), layer(PAR_B)])
    model, W = build(cfg, device)
    toks = tokens_of(90, seed=9)
    close(run_cut(replayer(model), "a", toks, [6]), oracle.forward(cfg, W, toks), TOL[torch.float32])


@pytest.mark.parametrize("device", DEVICES)
def test_greedy_generation_through_the_engine(device):
    """The framework's own entry point: scheduler, chunked prefill under a token budget, sampling (greedy), retirement."""
    model, W = build(HYBRID, device)
    eng = DynamicInferenceEngine(model, NullTokenizer(VOCAB - 1), max_sequence_length=128, num_blocks=64, block_size=4,
                                 max_tokens_per_step=16, max_requests=3)
    prompts = [tokens_of(21, seed=30), tokens_of(5, seed=31), tokens_of(33, seed=32), tokens_of(2, seed=33)]
    ids = [eng.add_request("", SamplingParams(num_tokens_to_generate=6, top_k=1), prompt_tokens=p) for p in prompts]
    while eng.has_unfinished_requests():
        eng.step()
    for rid, p in zip(ids, prompts):
        seq = list(p)
        for _ in range(6):
            logits = oracle.forward(HYBRID, W, seq)[-1]
            top2 = torch.topk(logits, 2).values
            if float(top2[0] - top2[1]) < 1e-3:
                break                                             # a close call is no test of the framework
            seq.append(int(torch.argmax(logits)))
        n = len(seq) - len(p)
        assert eng.completed[rid].generated_tokens.tolist()[:n] == seq[len(p):]


# 16-bit rounding may flip a close routing decision, which is no rounding error of the logits: these configurations route
# every token to all experts
SMOOTH = config_of([layer(PAR, MOE_C), layer(DELTA, DENSE), layer(PAR_B, MOE_C), layer(DELTA_B)])


def test_bfloat16_serving_stays_within_rounding():
    model, W = build(SMOOTH, "cpu", torch.bfloat16)
    toks = tokens_of(40, seed=12)
    want = oracle.forward(SMOOTH, {k: v.to(torch.bfloat16) for k, v in W.items()}, toks)
    close_in_16_bits(run_cut(replayer(model), "a", toks, [25, 2]), want)


@pytest.mark.gpu
def test_bfloat16_kernels_stay_within_rounding():
    cfg = config_of([layer(PAR_B, MOE_C), layer(DELTA_C, DENSE), layer(PAR_C, MOE_C)], width=64, side=8)
    model, W = build(cfg, "cuda", torch.bfloat16)
    toks = tokens_of(40, seed=12)
    want = oracle.forward(cfg, {k: v.to(torch.bfloat16) for k, v in W.items()}, toks)
    whole = run_cut(replayer(model), "a", toks, [40])
    close_in_16_bits(whole, want)
    close_in_16_bits(run_cut(replayer(model), "b", toks, [25, 2]), whole.double())


# ---------------------------------------------------------------------------------------------------------------------
# edges that random weights hide: one key that matters, at a window's edge, a page's border, far away; one bucket that matters
# ---------------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("dd,dv", [(6, 10), (32, 32)], ids=["narrow", "wide"])
@pytest.mark.parametrize("ctx_len,window,dist", [(5, 0, 4), (64, 16, 15), (64, 16, 16), (65, 64, 63), (65, 64, 64), (300, 0, 299),
                                                 (300, 128, 127), (300, 128, 128), (1200, 1000, 999), (1200, 1000, 1000), (40, 1, 0)])
def test_attention_sees_one_marked_key_just_inside_the_window_and_not_outside(ctx_len, window, dist, dd, dv, device):
    """All keys are small but one, ``dist`` positions before the last query, which matches the query strongly and whose
    value is marked: inside the window it dominates the output, outside it must leave no trace.  A bias table with small
    entries rides along.  Run as a whole prompt, with the last token decoded alone, and as a decoding batch; pages of 16, so
    the key also sits at page borders."""
    H, G, bs, B, D = 2, 1, 16, 8, 200.0
    g = torch.Generator().manual_seed(ctx_len + dist)
    k = torch.randn(ctx_len, G, dd, generator=g) * 0.01
    v = torch.randn(ctx_len, G, dv, generator=g) * 0.01
    q = torch.randn(ctx_len, H, dd, generator=g) * 0.01
    rel = torch.randn(B, H, generator=g) * 0.1
    j = ctx_len - 1 - dist
    k[j, 0] = 0.0
    k[j, 0, 0] = 8.0
    v[j, 0] = 5.0
    q[-1, :, 0] = 8.0
    want = oracle.window_attention(q[-1:].double(), k.double(), v.double(), 1.0, window, rel.double(), D, first=ctx_len - 1)[0]
    inside = window == 0 or dist < window
    assert (want[0, 0] > 4.9) == inside and (inside or want.abs().max() < 0.1)
    n_blocks = -(-ctx_len // bs)
    perm = torch.randperm(n_blocks, generator=g)
    table = perm.to(torch.int32).view(1, -1).to(device)
    kc, vc = torch.zeros(n_blocks * bs, G, dd), torch.zeros(n_blocks * bs, G, dv)
    pos = torch.arange(ctx_len)
    slots = perm[pos // bs] * bs + pos % bs
    kc[slots], vc[slots] = k, v
    bias = rel[distance_buckets(B, D, min(window, 201) if window else 201)].to(device)
    req = torch.zeros(ctx_len, dtype=torch.int32, device=device)
    lens = torch.arange(1, ctx_len + 1, dtype=torch.int32, device=device)
    whole = seqmix.window_attention_paged(q.to(device), kc.to(device), vc.to(device), table, req, lens, bs, 1.0, window, dist_bias=bias)
    close(whole[-1].view(H, dv), want, 1e-5)
    alone = seqmix.window_attention_paged(q[-1:].to(device), kc.to(device), vc.to(device), table, req[:1], lens[-1:], bs, 1.0, window,
                                          dist_bias=bias)
    close(alone[0].view(H, dv), want, 1e-5)
    split = seqmix.window_attention_paged(q[-1:].to(device), kc.to(device), vc.to(device), table, req[:1], lens[-1:], bs, 1.0, window,
                                          max_len=ctx_len, dist_bias=bias)
    close(split[0].view(H, dv), want, 1e-5)


@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("B,D,window", [(8, 20.0, 0), (8, 20.0, 30), (6, 40.0, 64), (16, 9.0, 12), (2, 3.0, 0)])
def test_one_loud_bucket_marks_exactly_its_distances(B, D, window, device):
    """Keys and queries are zero, so the weights come from the bias alone; value ``j`` is the one-hot of its position.  One
    bucket after the other gets a large entry: the last query's output then shows which distances fall into that bucket --
    the exact ones below ``B / 2``, the logarithmic ones above, everything from ``D`` on in the last -- as a prompt and as a
    decoded token."""
    ctx_len, bs = 48, 16
    q, k, v = torch.zeros(ctx_len, 1, 4), torch.zeros(ctx_len, 1, 4), torch.eye(ctx_len).view(ctx_len, 1, ctx_len)
    table, tok_req, tok_len = dense_pages(ctx_len, 1, device)
    table = torch.arange(ctx_len // bs, dtype=torch.int32, device=device).view(1, -1)
    lo = max(0, ctx_len - window) if window else 0
    for loud in range(B):
        rel = torch.zeros(B, 1)
        rel[loud, 0] = 30.0
        sat = int(D) + 2
        bias = rel[distance_buckets(B, D, min(window, sat) if window else sat)].to(device)
        members = [j for j in range(lo, ctx_len) if oracle.bucket(ctx_len - 1 - j, B, D) == loud]
        for got in (seqmix.window_attention_paged(q.to(device), k.to(device), v.to(device), table, tok_req, tok_len, bs, 1.0, window,
                                                  dist_bias=bias)[-1],
                    seqmix.window_attention_paged(q[-1:].to(device), k.to(device), v.to(device), table, tok_req[:1], tok_len[-1:], bs, 1.0,
                                                  window, dist_bias=bias, max_len=ctx_len)[0]):
            got = got.float().cpu()
            if members:
                assert sorted(torch.nonzero(got > 0.5 / len(members)).view(-1).tolist()) == members
            else:
                assert float(got.max()) < 0.5


@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["fp32", "bf16"])
@pytest.mark.parametrize("H,G,dd,dv,window", [(6, 2, 16, 16, 70), (5, 5, 20, 12, 0), (4, 2, 32, 24, 33), (12, 1, 8, 40, 100), (8, 1, 64, 64, 500)])
def test_decoding_batch_of_unequal_contexts_matches_prompts(H, G, dd, dv, window, dtype, device):
    """Three sequences of different lengths decode one token each in one call (the split path on the GPU); every result
    equals the last row of that sequence run as a prompt."""
    bs, B, D = 8, 12, 300.0
    lens = [3, 150, 517]
    g = torch.Generator().manual_seed(0)
    nb = [-(-n // bs) for n in lens]
    perm = torch.randperm(sum(nb), generator=g)
    table = torch.zeros(3, max(nb), dtype=torch.int32)
    kc, vc = torch.zeros(sum(nb) * bs, G, dd), torch.zeros(sum(nb) * bs, G, dv)
    rnd = lambda *sh: torch.randn(*sh, generator=g).to(dtype).float()  # noqa: E731
    rel = rnd(B, H)
    qs, wants, at = [], [], 0
    for r, n in enumerate(lens):
        table[r, :nb[r]] = perm[at:at + nb[r]].to(torch.int32)
        at += nb[r]
        k, v, q = rnd(n, G, dd), rnd(n, G, dv), rnd(1, H, dd)
        pos = torch.arange(n)
        slots = table[r].long()[pos // bs] * bs + pos % bs
        kc[slots], vc[slots] = k, v
        qs.append(q)
        wants.append(oracle.window_attention(q.double(), k.double(), v.double(), 0.25, window, rel.double(), D, first=n - 1)[0])
    d = lambda t: t.to(device)  # noqa: E731
    da = lambda t: t.to(device, dtype)  # noqa: E731
    bias = rel[distance_buckets(B, D, min(window, 302) if window else 302)]
    got = seqmix.window_attention_paged(da(torch.cat(qs)), da(kc), da(vc), d(table), d(torch.arange(3, dtype=torch.int32)),
                                        d(torch.tensor(lens, dtype=torch.int32)), bs, 0.25, window, max_len=max(lens), dist_bias=d(bias))
    for r in range(3):
        close(got[r].view(H, dv).float(), wants[r], 1e-5 if dtype == torch.float32 else 8e-3)


@pytest.mark.parametrize("device", DEVICES)
def test_first_tokens_see_only_what_exists(device):
    """With all scores equal the weights are uniform over the visible keys: token ``t`` averages ``min(t + 1, window)`` values."""
    T, window = 7, 4
    q, k = torch.zeros(T, 1, 4), torch.randn(T, 1, 4)
    v = torch.arange(T, dtype=torch.float32).view(T, 1, 1).repeat(1, 1, 4)
    table, tok_req, tok_len = dense_pages(T, 1, device)
    got = seqmix.window_attention_paged(q.to(device), k.to(device), v.to(device), table, tok_req, tok_len, T, 1.0, window)
    for t in range(T):
        n = min(t + 1, window)
        close(got[t], torch.full((4,), sum(range(t - n + 1, t + 1)) / n), 1e-6)


@pytest.mark.parametrize("device", DEVICES)
def test_memories_recall_an_early_write_after_hundreds_of_tokens_and_forget_by_their_decay(device):
    """Retention: the first token writes, later keys are orthogonal to the query, so the read-out is ``decay^t`` times the first
    value -- kept by a decay of one, lost by a small one -- whether the tokens come at once or in steps of one, two and many.
    Delta rule: the same with a decay input that keeps one head and empties the other; a second write to the same key replaces
    the value when beta is one."""
    T, H, dd, dv = 400, 2, 8, 4
    q, k, v = torch.zeros(T, H, dd), torch.zeros(T, H, dd), torch.zeros(T, H, dv)
    k[0, :, 0], v[0] = 1.0, torch.tensor([1.0, 2.0, 3.0, 4.0])
    k[1:, :, 1] = 1.0                                              # later writes go elsewhere
    v[1:] = 0.5
    q[:, :, 0] = 1.0
    decay = torch.tensor([1.0, 0.9])
    want = oracle.retention(q.double(), k.double(), v.double(), decay.double())
    assert float((want[-1, 0] - v[0, 0].double()).abs().max()) < 1e-9 and float(want[-1, 1].abs().max()) < 1e-12
    d = lambda t: t.to(device)  # noqa: E731
    state = torch.zeros(1, H, dd, dv, device=device)
    outs, at = [], 0
    for n in [1, 2, 1, 16, 17, 300, T]:
        n = min(n, T - at)
        if n:
            outs.append(seqmix.retention_scan(d(q[at:at + n]), d(k[at:at + n]), d(v[at:at + n]), d(decay), seqmix.PackedBatch([0, n], [0], device), state))
            at += n
    close(torch.cat(outs), want, 1e-6)
    # delta rule: unit keys already, decay per head and token
    log_g = torch.zeros(T, H)
    log_g[:, 1] = -0.2
    beta = torch.ones(T, H)
    k2, v2 = k.clone(), v.clone()
    k2[200, :, 0], k2[200, :, 1], v2[200] = 1.0, 0.0, torch.tensor([9.0, 8.0, 7.0, 6.0])       # overwrite the first key
    want = oracle.delta_rule(q.double(), k2.double(), v2.double(), torch.exp(log_g.double()), beta.double())
    assert float((want[199, 0] - v[0, 0].double()).abs().max()) < 1e-9 and float((want[-1, 0] - v2[200, 0].double()).abs().max()) < 1e-9
    state = torch.zeros(1, H, dd, dv, device=device)
    outs, at = [], 0
    for n in [1, 2, 1, 16, 17, 300, T]:
        n = min(n, T - at)
        if n:
            sl = slice(at, at + n)
            outs.append(seqmix.delta_rule_scan(d(q[sl]), d(k2[sl]), d(v2[sl]), d(log_g[sl]), d(beta[sl]), seqmix.PackedBatch([0, n], [0], device),
                                               state, None, 1.0))
            at += n
    close(torch.cat(outs), want, 1e-6)


@pytest.mark.parametrize("device", DEVICES)
def test_rotation_depends_on_the_position_not_on_the_step(device):
    """The same token decoded at position 700 of a sequence gets the angle of position 700: a query and a key written 3 tokens
    apart keep their relative angle wherever the pair sits, so the read-out of a pair (write, read) is the same at 0 and far out."""
    H, dd, dv = 1, 4, 2
    inv = seqmix.rotary_frequencies(4, 10.0).to(device)
    kq = torch.tensor([[[1.0, 2.0, -1.0, 0.5]]])
    val = torch.tensor([[[1.0, -2.0]]])
    outs = []
    for start in (0, 700):
        state = torch.zeros(1, H, dd, dv, device=device)
        pb = seqmix.PackedBatch([0, 1], [0], device)
        z = torch.zeros(1, H, dd, device=device)
        seqmix.retention_scan(z, kq.to(device), val.to(device), torch.ones(1, device=device), pb, state, torch.tensor([start], device=device), inv)
        outs.append(seqmix.retention_scan(kq.to(device), z, torch.zeros(1, H, dv, device=device), torch.ones(1, device=device), pb, state,
                                          torch.tensor([start + 3], device=device), inv).cpu())
    want = oracle.retention(oracle.rotate_half(torch.cat([torch.zeros(1, 1, 4), kq]).double(), [0, 3], 4, 10.0),
                            oracle.rotate_half(torch.cat([kq, torch.zeros(1, 1, 4)]).double(), [0, 3], 4, 10.0),
                            torch.cat([val, torch.zeros(1, 1, 2)]).double(), torch.ones(1).double())[1:]
    close(outs[0], want, 1e-5)
    close(outs[1], want, 2e-4)                                     # fp32 angles of a far position


@pytest.mark.parametrize("device", DEVICES)
def test_router_adds_its_bias_picks_the_largest_logits_and_weighs_them_alone(device):
    """Hand-made router rows: the bias changes the choice, the chosen experts are the top ones and their weights a softmax over
    the chosen (biased) logits."""
    cfg = config_of([layer(DELTA, MOE)], side=None)
    model, W = build(cfg, device)
    moe = model.decoder.layers[0].mlp
    h = torch.zeros(3, 1, 32, device=device)
    h[0, 0, 0], h[1, 0, 1], h[2, 0, 2] = 1.0, 1.0, 1.0
    bias = torch.tensor([0.0, 0.0, 2.5, 0.0, 0.0])
    with torch.no_grad():
        moe.router.weight.zero_()
        moe.router.weight[:, 0] = torch.tensor([0.0, 3.0, 1.0, 2.0, -1.0])
        moe.router.weight[:, 1] = torch.tensor([5.0, 0.0, 0.0, 0.0, 5.5])
        moe.router.weight[:, 2] = torch.tensor([-3.0, -2.0, -9.0, -8.0, -7.0])
        moe.router.logit_bias.copy_(bias)
        probs, rmap = moe.router(h)
    probs, rmap = probs.view(3, 5).cpu(), rmap.view(3, 5).cpu()
    assert rmap.tolist() == [[False, True, True, False, False], [True, False, False, False, True], [True, True, False, False, False]]
    for row, (i, j) in zip(range(3), ((2, 1), (4, 0), (1, 0))):
        z = moe.router.weight[:, row].cpu().double() + bias.double()
        want = torch.softmax(torch.stack([z[i], z[j]]), 0)
        close(torch.stack([probs[row, i], probs[row, j]]), want, 1e-6)


def test_config_reads_its_keys_and_rejects_bad_values():
    c = NunosunConfig.from_dict(HYBRID)
    assert (c.canon_taps, c.side_dim, c.logit_scale, len(c.layers)) == (3, 6, 0.5, 5)
    c = NunosunConfig.from_dict(config_of([layer(DELTA)], taps=None, side=None, logit_scale=None))
    assert (c.canon_taps, c.side_dim, c.logit_scale) == (0, 0, 1.0)
    bad = config_of([layer(PAR)])
    bad["layers"][0]["type"] = "other"
    with pytest.raises(ValueError):
        NunosunConfig.from_dict(bad)
    bad = config_of([layer(DELTA, {"kind": "other"})])
    with pytest.raises(ValueError):
        NunosunConfig.from_dict(bad)
    filled = shapes_into_config(config_of([layer(PAR)]), {"l0.mix.left.rel": (14, 4)})
    assert filled["layers"][0]["mixer"]["left"]["bias_buckets"] == 14


# ---------------------------------------------------------------------------------------------------------------------
# a model folder through the registry, the trace runner and its command line
# ---------------------------------------------------------------------------------------------------------------------
def write_safetensors(path, tensors):
    header, blobs, at = {}, [], 0
    for name, t in tensors.items():
        raw = t.contiguous().view(torch.uint8).numpy().tobytes() if t.dtype != torch.bfloat16 else \
            t.contiguous().view(torch.int16).numpy().tobytes()
        code = {torch.bfloat16: "BF16", torch.float32: "F32"}[t.dtype]
        header[name] = {"dtype": code, "shape": list(t.shape), "data_offsets": [at, at + len(raw)]}
        blobs.append(raw)
        at += len(raw)
    hj = json.dumps(header).encode()
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hj)) + hj + b"".join(blobs))


def test_model_folder_through_registry_and_trace_runner_command_line(tmp_path):
    from megatronapp_b200.models.registry import architectures, build_model_from_dir

    assert "nunosun" in architectures()
    cfg = config_of([layer(PAR, MOE), layer(DELTA, DENSE_B)])
    W = {k: v.to(torch.bfloat16) for k, v in oracle.random_weights(cfg, 5, bias_buckets=9).items()}
    folder = tmp_path / "model"
    folder.mkdir()
    (folder / "config.json").write_text(json.dumps(cfg))
    write_safetensors(str(folder / "model.safetensors"), W)
    model = build_model_from_dir(str(folder), torch.float32, "cpu")
    assert model.decoder.layers[0].mixer.left.bias_buckets == 9                    # read from the tensor's shape
    toks = tokens_of(12, seed=3)
    want = oracle.forward(cfg, W, toks)
    close(run_cut(replayer(model), "a", toks, [12]), want, TOL[torch.float32])
    steps = [{"step": 0, "entries": [{"id": "x", "tokens": toks[:9], "want": [0, 8]}], "end": []},
             {"step": 1, "entries": [{"id": "x", "tokens": toks[9:10], "want": []}], "end": []},
             {"step": 2, "entries": [{"id": "x", "tokens": toks[10:], "want": [1]}], "end": ["x"]}]
    out = tmp_path / "out"
    exe = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "bin", "trace_run")
    r = subprocess.run([sys.executable, exe, "--model", str(folder), "--dtype", "float32", "--out", str(out), "--max-tokens", "64",
                        "--device", "cpu"], input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True,
                       timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    assert [l for l in r.stdout.splitlines() if l.startswith("done")] == ["done 0", "done 1", "done 2"]
    assert not (out / "1.f32").exists()
    got0 = torch.frombuffer(bytearray((out / "0.f32").read_bytes()), dtype=torch.float32).view(2, -1)
    got2 = torch.frombuffer(bytearray((out / "2.f32").read_bytes()), dtype=torch.float32).view(1, -1)
    close(got0, want[[0, 8]], TOL[torch.float32])
    close(got2, want[[11]], TOL[torch.float32])
    # the generation command line on the same folder: greedy tokens of the oracle (a close call is no test)
    prompt, gen = toks[:7], []
    for _ in range(4):
        top2 = torch.topk(oracle.forward(cfg, W, prompt + gen)[-1], 2)
        if float(top2.values[0] - top2.values[1]) < 1e-3:
            break
        gen.append(int(top2.indices[0]))
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    r = subprocess.run([sys.executable, os.path.join(root, "tools", "run_text_generation_server.py"), "--model-dir", str(folder),
                        "--dtype", "float32", "--prompts", " ".join(map(str, prompt)), "--num-tokens-to-generate", "4"],
                       capture_output=True, text=True, env=dict(os.environ, CUDA_VISIBLE_DEVICES=""), timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    said = r.stdout.strip().splitlines()[-1].split("-> ")[-1].strip("'\"").split()
    assert [int(t) for t in said][:len(gen)] == gen
