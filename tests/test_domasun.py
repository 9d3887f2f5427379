"""Domasun models in the framework against a plain, slow evaluation of the design's equations (``domasun_oracle``).

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

import domasun_oracle as oracle
from megatronapp_b200.data.tokenizer import NullTokenizer
from megatronapp_b200.inference import DynamicInferenceEngine, SamplingParams
from megatronapp_b200.inference.trace import TraceReplayer
from megatronapp_b200.models.domasun import DomasunConfig, DomasunModel
from megatronapp_b200.models.domasun.loader import load_domasun_weights
from megatronapp_b200.ops import seqmix
from megatronapp_b200.parallel import state as ps
from megatronapp_b200.transformer.mixed_head_attention import dense_pages

DEVICES = ["cpu", pytest.param("cuda", marks=pytest.mark.gpu)]
VOCAB = 70

LEFT = {"heads": 6, "kv_heads": 2, "dim": 8, "vdim": 8, "scale": 0.3, "mask": {"size": 11}}
LEFT_B = {"heads": 3, "kv_heads": 3, "dim": 20, "vdim": 20, "scale": 0.2, "mask": {"size": 5}}
LEFT_C = {"heads": 4, "kv_heads": 1, "dim": 36, "vdim": 36, "scale": 0.15, "mask": {"size": 64}}
RIGHT = {"inner": 24, "state": 5, "dt_rank": 3, "conv": 3}
RIGHT_B = {"inner": 40, "state": 16, "dt_rank": 8, "conv": 2}
RIGHT_C = {"inner": 36, "state": 33, "dt_rank": 4, "conv": 5}
PAR = {"type": "parallel", "mixer": {"left": LEFT, "right": RIGHT, "left_scale": 0.7, "right_scale": 1.3}}
PAR_B = {"type": "parallel", "mixer": {"left": LEFT_B, "right": RIGHT_B, "left_scale": 1.0, "right_scale": 1.0}}
PAR_C = {"type": "parallel", "mixer": {"left": LEFT_C, "right": RIGHT_C, "left_scale": 1.2, "right_scale": 0.5}}
ONLY_LEFT = {"type": "parallel", "mixer": {"left": LEFT, "right": RIGHT, "left_scale": 1.0, "right_scale": 0.0}}
ONLY_RIGHT = {"type": "parallel", "mixer": {"left": LEFT, "right": RIGHT, "left_scale": 0.0, "right_scale": 1.0}}
MOE = {"kind": "moe", "expert": {"ff": 16, "limit": 0.9}, "router": {"experts": 5, "top": 2}, "shared": {"ff": 24, "limit": 0.6}}
MOE_B = {"kind": "moe", "expert": {"ff": 8, "limit": 3.0}, "router": {"experts": 3, "top": 1}}                      # top 1, no shared expert
MOE_C = {"kind": "moe", "expert": {"ff": 24, "limit": 1.5}, "router": {"experts": 4, "top": 4}, "shared": {"ff": 8, "limit": 2.0}}


def layer(spec, mlp=None):
    l = copy.deepcopy(spec)
    l["mlp"] = copy.deepcopy(mlp)
    return l


def config_of(layers, width=32, vocab=VOCAB, eps=1e-5, streams=3, loop=None, softcap=9.0):
    cfg = {"architecture": "Domasun", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}
    if streams is not None:
        cfg["streams"] = streams
    if loop is not None:
        cfg["loop"] = loop
    if softcap is not None:
        cfg["logit_softcap"] = softcap
    return cfg


HYBRID = config_of([layer(PAR, MOE), layer(PAR_B, MOE_B), layer(PAR_C), layer(PAR, MOE_C)], loop={"start": 1, "stop": 3, "times": 2})


def build(cfg, device, dtype=torch.float32, seed=0, weights=None):
    if not ps.model_parallel_is_initialized():
        ps.initialize_model_parallel(1, 1)
    W = weights if weights is not None else oracle.random_weights(cfg, seed)
    dcfg = DomasunConfig.from_dict(copy.deepcopy(cfg))
    model = DomasunModel(dcfg, dcfg.base_transformer_config(dtype, use_cpu_initialization=True, perform_initialization=False))
    load_domasun_weights(model, W)
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


# ---------------------------------------------------------------------------------------------------------------------
# every mechanism alone: one layer, whole prompt and cut prompt
# ---------------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("spec,streams", [(layer(ONLY_LEFT), 3), (layer(ONLY_RIGHT), 3), (layer(PAR), None), (layer(PAR), 1), (layer(PAR_B), 2),
                                          (layer(PAR_C), 4), (layer(ONLY_RIGHT, MOE), 3), (layer(ONLY_RIGHT, MOE_B), None),
                                          (layer(ONLY_LEFT, MOE_C), 2)],
                         ids=["attention", "scan", "plain_residual", "one_stream", "two_streams", "four_streams_wide_window", "moe",
                              "moe_top1_no_shared", "moe_all_experts"])
def test_single_mechanism_matches_oracle(spec, streams, device):
    cfg = config_of([spec], streams=streams)
    model, W = build(cfg, device)
    toks = tokens_of(37)
    want, layers = oracle.forward(cfg, W, toks, return_layers=True)
    seen = []
    model.decoder.tap = lambda i, x: seen.append(x.detach().float().cpu().clone())
    rp = replayer(model)
    close(run_cut(rp, "a", toks, [len(toks)]), want, TOL[torch.float32])
    close(seen[0].view(len(toks), -1), layers[0], TOL[torch.float32])
    model.decoder.tap = None
    close(run_cut(rp, "b", toks, [17, 2, 16]), want, TOL[torch.float32])


def test_whole_sequence_forward_without_a_context_and_without_softcap():
    """The training-style call (``[b, s]`` ids, no inference context) runs the same mixers from zero state."""
    for cfg in (HYBRID, config_of([layer(PAR_B, MOE), layer(PAR)], streams=None, softcap=None)):
        model, W = build(cfg, "cpu")
        a, b = tokens_of(21, seed=1), tokens_of(21, seed=2)
        out = model(torch.tensor([a, b]), None, None)
        close(out[0], oracle.forward(cfg, W, a), TOL[torch.float32])
        close(out[1], oracle.forward(cfg, W, b), TOL[torch.float32])


@pytest.mark.parametrize("device", DEVICES)
def test_ops_match_the_oracle_functions(device):
    """The op level: stream update + norm, sinusoidal positions, per-head norm, windowed attention, convolution with bias,
    selective scan -- each against the oracle's function for that mechanism."""
    g = torch.Generator().manual_seed(3)
    rnd = lambda *s: torch.randn(*s, generator=g)  # noqa: E731
    T, S, Wd = 9, 3, 20
    # streams: update by two branches, then read + layer norm
    x, a, b, ba, ls = rnd(T, S, Wd), rnd(T, Wd), rnd(T, Wd), rnd(Wd), rnd(Wd)
    mix, outc, inp, w, beta = rnd(S, S), rnd(S), rnd(S), rnd(Wd), rnd(Wd)
    y = ls * (0.7 * (a + ba) + 1.3 * b)
    want_x = torch.einsum("st,nsw->ntw", mix.double(), x.double()) + outc.double().view(1, S, 1) * y.double().unsqueeze(1)
    want_h = oracle.layer_norm(torch.einsum("s,nsw->nw", inp.double(), want_x), w.double(), beta.double(), 1e-5)
    d = lambda t: t.to(device)  # noqa: E731
    gx, gh = seqmix.stream_mix_norm(d(x.clone()), d(a), d(b), d(ba), d(ls), 0.7, 1.3, d(mix), d(outc), d(inp), d(w), d(beta), 1e-5)
    close(gx, want_x, 1e-5), close(gh, want_h, 1e-5)
    # sinusoidal positions
    pos = torch.tensor([0, 1, 2, 500, 501, 3, 4000, 7, 8])
    e = seqmix.add_sinusoid(d(torch.zeros(T, Wd)), d(pos), d(torch.tensor([10000.0 ** (-2.0 * i / Wd) for i in range(Wd // 2)])))
    for n, p in enumerate(pos.tolist()):
        close(e[n], oracle.sinusoid(1, Wd, first=p)[0], 5e-4)
    # per-head norm of a strided view
    big = rnd(T, 4 * 6 + 5)
    hw = rnd(6)
    close(seqmix.head_rms_norm(d(big)[:, 3:27].view(T, 4, 6), d(hw), 1e-5), oracle.head_rms(big[:, 3:27].reshape(T, 4, 6).double(), hw.double(), 1e-5), 1e-5)
    # attention: two sequences of 9 tokens, window 4, H = 4 over G = 2
    H, G, dd = 4, 2, 6
    q, k, v, gate = rnd(2 * T, H, dd), rnd(2 * T, G, dd), rnd(2 * T, G, dd), rnd(2 * T, H)
    table, tok_req, tok_len = dense_pages(T, 2, device)
    for window, sink in ((4, True), (0, True), (3, False)):
        got = seqmix.window_attention_paged(d(q), d(k), d(v), table, tok_req, tok_len, T, 0.4, window, d(torch.tensor(oracle.slopes(H))),
                                            sink, d(gate), 1.5)
        for r in range(2):
            sl = slice(r * T, (r + 1) * T)
            want = oracle.window_attention(q[sl].double(), k[sl].double(), v[sl].double(), 0.4, window, oracle.slopes(H), sink)
            want = want * torch.sigmoid(gate[sl].double()).unsqueeze(-1) * 1.5
            close(got[sl].view(T, H, dd), want, 1e-5)
    # convolution with bias + selective scan, two sequences, carried state
    C, N, taps = 10, 5, 3
    u, cw, cb = rnd(2 * T, C), rnd(C, taps), rnd(C)
    pb = seqmix.PackedBatch.dense(T, 2, device)
    win = torch.zeros(2, taps - 1, C, device=device)
    got = seqmix.causal_conv_silu(d(u), d(cw), pb, win, d(cb))
    for r in range(2):
        close(got[r * T:(r + 1) * T], oracle.silu(oracle.causal_conv(u[r * T:(r + 1) * T].double(), cw.double(), cb.double())), 1e-5)
    xs, dtp, B, Cm, A_log, D, z, dtb = rnd(2 * T, C), rnd(2 * T, C), rnd(2 * T, N), rnd(2 * T, N), rnd(C, N) * 0.5, rnd(C), rnd(2 * T, C), rnd(C)
    state = torch.zeros(2, C, N, device=device)
    got = seqmix.selective_scan(d(xs), d(dtp), d(B), d(Cm), d(A_log), d(D), pb, state, d(z), d(dtb), 0.9)
    for r in range(2):
        sl = slice(r * T, (r + 1) * T)
        dt = torch.log1p(torch.exp(dtp[sl].double() + dtb.double()))
        want = oracle.selective_scan(xs[sl].double(), dt, -torch.exp(A_log.double()), B[sl].double(), Cm[sl].double(), D.double())
        close(got[sl], want * oracle.silu(z[sl].double()) * 0.9, 1e-5)


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
    """kv heads == heads, one kv head, one head, one expert, two taps, one tap, a state of one, rank one, a loop over
    everything, a loop that runs once, no loop, scales of one, a window of one and a window longer than the prompt, eleven streams."""
    left = {"heads": 1, "kv_heads": 1, "dim": 12, "vdim": 12, "scale": 1.0, "mask": {"size": 1}}
    right = {"inner": 6, "state": 1, "dt_rank": 1, "conv": 1}
    one = {"type": "parallel", "mixer": {"left": left, "right": right, "left_scale": 1.0, "right_scale": 1.0}}
    moe1 = {"kind": "moe", "expert": {"ff": 4, "limit": 1.0}, "router": {"experts": 1, "top": 1}, "shared": {"ff": 4, "limit": 1.0}}
    for cfg in (config_of([layer(one, moe1), layer(PAR_C, MOE)], width=24, loop={"start": 0, "stop": 2, "times": 3}, streams=2),
                config_of([layer(PAR_B, MOE_B), layer(one)], width=40, loop={"start": 1, "stop": 2, "times": 1}, streams=1, softcap=None),
                config_of([layer(PAR_C, MOE_C)], width=16, eps=1e-3, streams=5),
                config_of([layer(PAR_B, MOE_B)], width=20, streams=11)):
        model, W = build(cfg, device, seed=11)
        toks = tokens_of(29, seed=8)
        close(run_cut(replayer(model), "a", toks, [13, 2, 9]), oracle.forward(cfg, W, toks), TOL[torch.float32])


@pytest.mark.parametrize("device", DEVICES)
def test_long_decoding_passes_the_window_over_decoded_tokens(device):
    cfg = config_of([layer(PAR, MOE), layer(PAR_B)], loop={"start": 0, "stop": 1, "times": 2})
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
SMOOTH = config_of([layer(PAR, MOE_C), layer(PAR_B, MOE_C), layer(PAR_C)], loop={"start": 0, "stop": 2, "times": 2})


def test_bfloat16_serving_stays_within_rounding():
    model, W = build(SMOOTH, "cpu", torch.bfloat16)
    toks = tokens_of(40, seed=12)
    want = oracle.forward(SMOOTH, {k: v.to(torch.bfloat16) for k, v in W.items()}, toks)
    close(run_cut(replayer(model), "a", toks, [25, 2]), want, TOL[torch.bfloat16])


@pytest.mark.gpu
def test_bfloat16_kernels_stay_within_rounding():
    cfg = config_of([layer(PAR_B, MOE_C), layer(PAR_C, MOE_C)], width=64)
    model, W = build(cfg, "cuda", torch.bfloat16)
    toks = tokens_of(40, seed=12)
    want = oracle.forward(cfg, {k: v.to(torch.bfloat16) for k, v in W.items()}, toks)
    whole = run_cut(replayer(model), "a", toks, [40])
    close(whole, want, TOL[torch.bfloat16])
    close(run_cut(replayer(model), "b", toks, [25, 2]), whole.double(), TOL[torch.bfloat16])


# ---------------------------------------------------------------------------------------------------------------------
# edges that random weights hide: one key that matters, at a window's edge, a page's border, far away
# ---------------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("dd", [6, 32], ids=["narrow", "wide"])
@pytest.mark.parametrize("ctx_len,window,dist", [(5, 0, 4), (64, 16, 15), (64, 16, 16), (65, 64, 63), (65, 64, 64), (300, 0, 299),
                                                 (300, 128, 127), (300, 128, 128), (1200, 1000, 999), (1200, 1000, 1000), (40, 1, 0)])
def test_attention_sees_one_marked_key_just_inside_the_window_and_not_outside(ctx_len, window, dist, dd, device):
    """All keys are small but one, ``dist`` positions before the last query, which matches the query strongly and whose
    value is marked: inside the window it dominates the output (up to the sink's share), outside it must leave no trace.
    Run as a whole prompt and with the last token decoded alone; pages of 16, so the key also sits at page borders."""
    H, G, bs = 2, 1, 16
    g = torch.Generator().manual_seed(ctx_len + dist)
    k = torch.randn(ctx_len, G, dd, generator=g) * 0.01
    v = torch.randn(ctx_len, G, dd, generator=g) * 0.01
    q = torch.randn(ctx_len, H, dd, generator=g) * 0.01
    j = ctx_len - 1 - dist
    k[j, 0] = 0.0
    k[j, 0, 0] = 8.0
    v[j, 0] = 5.0
    q[-1, :, 0] = 8.0
    slope = [0.0, 0.01]
    want = oracle.window_attention(q[-1:].double(), k.double(), v.double(), 1.0, window, slope, True, first=ctx_len - 1)[0]
    inside = window == 0 or dist < window
    assert (want[0, 0] > 4.9) == inside and (inside or want.abs().max() < 0.1)
    n_blocks = -(-ctx_len // bs)
    perm = torch.randperm(n_blocks, generator=g)
    table = perm.to(torch.int32).view(1, -1).to(device)
    kc, vc = torch.zeros(n_blocks * bs, G, dd), torch.zeros(n_blocks * bs, G, dd)
    pos = torch.arange(ctx_len)
    slots = perm[pos // bs] * bs + pos % bs
    kc[slots], vc[slots] = k, v
    sl = torch.tensor(slope)
    req = torch.zeros(ctx_len, dtype=torch.int32, device=device)
    lens = torch.arange(1, ctx_len + 1, dtype=torch.int32, device=device)
    whole = seqmix.window_attention_paged(q.to(device), kc.to(device), vc.to(device), table, req, lens, bs, 1.0, window, sl.to(device), True)
    close(whole[-1].view(H, dd), want, 1e-5)
    alone = seqmix.window_attention_paged(q[-1:].to(device), kc.to(device), vc.to(device), table, req[:1], lens[-1:], bs, 1.0, window,
                                          sl.to(device), True)
    close(alone[0].view(H, dd), want, 1e-5)
    # a decoding batch (one token per sequence, the longest context known): the keys are split over several CTAs on the GPU
    split = seqmix.window_attention_paged(q[-1:].to(device), kc.to(device), vc.to(device), table, req[:1], lens[-1:], bs, 1.0, window,
                                          sl.to(device), True, max_len=ctx_len)
    close(split[0].view(H, dd), want, 1e-5)


@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["fp32", "bf16"])
@pytest.mark.parametrize("H,G,dd,dv,window,sink", [(6, 2, 16, 16, 70, True), (5, 5, 20, 20, 0, True), (4, 2, 32, 24, 33, False),
                                                   (12, 1, 8, 40, 100, True), (8, 1, 64, 64, 500, True), (3, 1, 36, 36, 64, False)])
def test_decoding_batch_of_unequal_contexts_splits_keys_and_matches_prompts(H, G, dd, dv, window, sink, dtype, device):
    """Three sequences of different lengths decode one token each in one call (the split path on the GPU); every result
    equals the last row of that sequence run as a prompt.  Gate, slopes; one, two, three, eight and twelve heads per kv head,
    head sizes with and without 16-byte rows, values narrower and wider than keys, with and without window and sink."""
    bs = 8
    lens = [3, 150, 517]
    g = torch.Generator().manual_seed(0)
    nb = [-(-n // bs) for n in lens]
    perm = torch.randperm(sum(nb), generator=g)
    table = torch.zeros(3, max(nb), dtype=torch.int32)
    kc, vc = torch.zeros(sum(nb) * bs, G, dd), torch.zeros(sum(nb) * bs, G, dv)
    qs, gates, wants, at = [], [], [], 0
    slope = oracle.slopes(H)
    rnd = lambda *sh: torch.randn(*sh, generator=g).to(dtype).float()  # noqa: E731
    for r, n in enumerate(lens):
        table[r, :nb[r]] = perm[at:at + nb[r]].to(torch.int32)
        at += nb[r]
        k, v, q, gt = rnd(n, G, dd), rnd(n, G, dv), rnd(1, H, dd), rnd(1, H)
        pos = torch.arange(n)
        slots = table[r].long()[pos // bs] * bs + pos % bs
        kc[slots], vc[slots] = k, v
        qs.append(q), gates.append(gt)
        o = oracle.window_attention(q.double(), k.double(), v.double(), 0.25, window, slope, sink, first=n - 1)[0]
        wants.append(o * torch.sigmoid(gt[0].double()).unsqueeze(-1))
    d = lambda t: t.to(device)  # noqa: E731
    da = lambda t: t.to(device, dtype)  # noqa: E731
    got = seqmix.window_attention_paged(da(torch.cat(qs)), da(kc), da(vc), d(table), d(torch.arange(3, dtype=torch.int32)),
                                        d(torch.tensor(lens, dtype=torch.int32)), bs, 0.25, window, d(torch.tensor(slope)), sink,
                                        da(torch.cat(gates)), 1.0, max(lens))
    for r in range(3):
        close(got[r].view(H, dv).float(), wants[r], 1e-5 if dtype == torch.float32 else 8e-3)


@pytest.mark.parametrize("device", DEVICES)
def test_sink_takes_its_share_and_first_tokens_see_only_themselves(device):
    """With all scores at zero the weights are 1 / (n + 1): the first token keeps half of its value, the second two thirds of
    the mean, and so on up to the window."""
    T, window = 7, 4
    q = torch.zeros(T, 1, 4)
    k = torch.randn(T, 1, 4)
    v = torch.ones(T, 1, 4)
    table, tok_req, tok_len = dense_pages(T, 1, device)
    got = seqmix.window_attention_paged(q.to(device), k.to(device), v.to(device), table, tok_req, tok_len, T, 1.0, window, None, True)
    for t in range(T):
        n = min(t + 1, window)
        close(got[t], torch.full((4,), n / (n + 1.0)), 1e-6)
    got = seqmix.window_attention_paged(q.to(device), k.to(device), v.to(device), table, tok_req, tok_len, T, 1.0, window, None, False)
    close(got, torch.ones(T, 4), 1e-6)


@pytest.mark.parametrize("device", DEVICES)
def test_scan_recalls_an_early_write_after_hundreds_of_tokens_and_the_convolution_crosses_steps(device):
    """A channel that barely decays keeps what the first token wrote; fed in steps of one, two and many tokens the scan and
    the convolution window give the same result as in one piece."""
    T, C, N, taps = 400, 6, 3, 4
    g = torch.Generator().manual_seed(1)
    x = torch.zeros(T, C)
    x[0] = 3.0
    dt_pre = torch.full((T, C), -2.0)
    A_log = torch.full((C, N), -9.0)
    A_log[3:] = 1.0                                                  # channels 3.. forget quickly
    B, Cm, D = torch.ones(T, N), torch.ones(T, N), torch.zeros(C)
    dt = torch.log1p(torch.exp(dt_pre.double()))
    want = oracle.selective_scan(x.double(), dt, -torch.exp(A_log.double()), B.double(), Cm.double(), D.double())
    assert want[-1, 0] > 0.9 * want[0, 0] > 0 and want[-1, 4].abs() < 1e-6
    d = lambda t: t.to(device)  # noqa: E731
    state = torch.zeros(1, C, N, device=device)
    outs, at = [], 0
    for n in [1, 2, 1, 16, 17, 300]:
        n = min(n, T - at)
        pb = seqmix.PackedBatch([0, n], [0], device)
        sl = slice(at, at + n)
        outs.append(seqmix.selective_scan(d(x[sl]), d(dt_pre[sl]), d(B[sl]), d(Cm[sl]), d(A_log), d(D), pb, state))
        at += n
    pb = seqmix.PackedBatch([0, T - at], [0], device)
    outs.append(seqmix.selective_scan(d(x[at:]), d(dt_pre[at:]), d(B[at:]), d(Cm[at:]), d(A_log), d(D), pb, state))
    close(torch.cat(outs), want, 1e-5)
    u, cw, cb = torch.randn(40, C, generator=g), torch.randn(C, taps, generator=g), torch.randn(C, generator=g)
    want = oracle.causal_conv(u.double(), cw.double(), cb.double())
    win = torch.zeros(1, taps - 1, C, device=device)
    outs, at = [], 0
    for n in [1, 1, 2, 1, 2, 5, 28]:
        outs.append(seqmix.causal_conv(d(u[at:at + n]), d(cw), seqmix.PackedBatch([0, n], [0], device), win, bias=d(cb)))
        at += n
    close(torch.cat(outs), want, 1e-5)


@pytest.mark.parametrize("device", DEVICES)
def test_router_picks_the_largest_logits_and_weighs_them_alone(device):
    """Hand-made router rows: the chosen experts are the top ones and their weights a softmax over the chosen logits."""
    cfg = config_of([layer(ONLY_RIGHT, MOE)], streams=None)
    model, W = build(cfg, device)
    moe = model.decoder.layers[0].mlp
    h = torch.zeros(3, 1, 32, device=device)
    h[0, 0, 0], h[1, 0, 1], h[2, 0, 2] = 1.0, 1.0, 1.0
    with torch.no_grad():
        moe.router.weight.zero_()
        moe.router.weight[:, 0] = torch.tensor([0.0, 3.0, 1.0, 2.0, -1.0])
        moe.router.weight[:, 1] = torch.tensor([5.0, 0.0, 0.0, 0.0, 5.5])
        moe.router.weight[:, 2] = torch.tensor([-3.0, -2.0, -9.0, -8.0, -7.0])
        probs, rmap = moe.router(h)
    probs, rmap = probs.view(3, 5).cpu(), rmap.view(3, 5).cpu()
    assert rmap.tolist() == [[False, True, False, True, False], [True, False, False, False, True], [True, True, False, False, False]]
    for row, (i, j) in zip(range(3), ((1, 3), (4, 0), (1, 0))):
        z = moe.router.weight[:, row].cpu().double()
        want = torch.softmax(torch.stack([z[i], z[j]]), 0)
        close(torch.stack([probs[row, i], probs[row, j]]), want, 1e-6)


def test_config_reads_loop_streams_and_rejects_bad_values():
    d = DomasunConfig.from_dict(HYBRID)
    assert d.runs() == [0, 1, 2, 1, 2, 3] and d.streams == 3
    assert DomasunConfig.from_dict(config_of([layer(PAR)], streams=None)).streams is None
    with pytest.raises(ValueError):
        DomasunConfig.from_dict(config_of([layer(PAR)], loop={"start": 1, "stop": 3, "times": 2}))
    bad = config_of([layer(PAR)])
    bad["layers"][0]["type"] = "other"
    with pytest.raises(ValueError):
        DomasunConfig.from_dict(bad)


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

    assert "domasun" in architectures()
    cfg = config_of([layer(PAR, MOE), layer(PAR_B)], loop={"start": 0, "stop": 1, "times": 2})
    W = {k: v.to(torch.bfloat16) for k, v in oracle.random_weights(cfg, 5).items()}
    folder = tmp_path / "model"
    folder.mkdir()
    (folder / "config.json").write_text(json.dumps(cfg))
    write_safetensors(str(folder / "model.safetensors"), W)
    model = build_model_from_dir(str(folder), torch.float32, "cpu")
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
