"""Serving benchmark of the hybrid (Zikunex) design beside the closest existing model, a GPT decoder with grouped-query
attention and the same feed-forwards, both through ``DynamicInferenceEngine.forward_tokens`` (``bench.py --serving``);
with ``--serving-design lerorax`` the Lerorax design beside its closest existing model, Zikunex, at equal width, depth and
head sizes, and the Lerorax kernels beside their like kernels; with ``--serving-design domasun`` the Domasun design beside its
closest existing model, Lerorax (two mixers side by side on a paged attention and a recurrent memory), and its kernels
beside their like kernels; with ``--serving-design nunosun`` the Nunosun design beside its closest existing model, Domasun
(sliding-window attention beside a recurrent memory, mixtures of experts), and its kernels beside their like kernels.

Two parts, random weights, bf16:

* model level: prefill (a few long prompts in one step) and decode (many requests, one token each, against a filled
  cache) in tokens/s, for both models at equal width, depth, head count and feed-forward sizes;
* kernel level: every kernel of the new design alone, with its achieved fraction of the roofline (measured copy
  bandwidth for the memory-bound ones, fp32 FMA rate for the sequential scans' prefill), next to the like kernel of the
  existing models (paged GQA attention, the fused LayerNorm/RMSNorm kernel, the Mamba SSD scan).

Timing: CUDA events on the launching stream, warm-up first, an L2-sized buffer rewritten between timed kernel launches.
"""
from __future__ import annotations

import json
import os
import time

import torch

SIZES = {
    # width, layers, heads, head dim, latent ranks (kv, q), dense ff, experts, expert ff, top, shared ff, vocab
    "small": dict(width=1024, layers=4, heads=8, dim=128, kv_rank=256, q_rank=384, ff=4096, experts=8, expert_ff=512, top=2,
                  shared_ff=1024, vocab=32000),
    "medium": dict(width=2048, layers=8, heads=16, dim=128, kv_rank=512, q_rank=768, ff=8192, experts=16, expert_ff=1024, top=4,
                   shared_ff=2048, vocab=32000),
}


def _peaks():
    p = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            d = json.load(f)
        return float(d["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


def zikunex_config(s):
    moe = {"kind": "moe", "expert": {"ff": s["expert_ff"]},
           "router": {"experts": s["experts"], "top": s["top"], "groups": {"count": 4, "keep": 2}}, "shared": {"ff": s["shared_ff"]}}
    dense = {"kind": "dense", "ff": s["ff"]}
    lat = {"heads": s["heads"], "dim": s["dim"], "vdim": s["dim"], "kv_rank": s["kv_rank"], "q_rank": s["q_rank"],
           "scale": s["dim"] ** -0.5}
    pattern = [("mlstm", {"heads": s["heads"], "dim": s["dim"], "vdim": s["dim"], "gate_cap": 15.0}, dense),
               ("latent_attention", lat, moe),
               ("channel_delta", {"heads": s["heads"], "kv_heads": s["heads"] // 2, "dim": s["dim"], "vdim": s["dim"], "conv": 4,
                                  "decay_rank": 64, "gate_rank": 64}, moe),
               ("latent_attention", dict(lat, kv_from=1), moe)]
    layers = []
    for i in range(s["layers"]):
        t, mx, mlp = pattern[i % 4]
        mx = dict(mx)
        if "kv_from" in mx:
            mx["kv_from"] = i - 2
        layers.append({"type": t, "mixer": mx, "mlp": mlp})
    return {"architecture": "Zikunex", "vocab": s["vocab"], "width": s["width"], "norm": {"eps": 1e-5}, "embedding": {"scale": 1.0},
            "layers": layers}


def build_zikunex(s, device):
    from .models.zikunex import ZikunexConfig, ZikunexModel
    from .parallel import state as ps

    if not ps.model_parallel_is_initialized():
        ps.initialize_model_parallel(1, 1)
    zcfg = ZikunexConfig.from_dict(zikunex_config(s))
    base = zcfg.base_transformer_config(torch.bfloat16, use_cpu_initialization=False)
    return ZikunexModel(zcfg, base).to(device).eval()


def build_gpt(s, device):
    """The closest existing model: GQA attention with rotary positions, RMSNorm, the same MoE / dense feed-forward sizes
    (3 of 4 layers MoE, like the hybrid), squared-ReLU experts, a shared expert."""
    from .config.transformer_config import TransformerConfig
    from .models.gpt.gpt_layer_specs import get_gpt_decoder_block_spec
    from .models.gpt.gpt_model import GPTModel
    from .parallel import state as ps
    from .transformer.mlp import squared_relu

    if not ps.model_parallel_is_initialized():
        ps.initialize_model_parallel(1, 1)
    cfg = TransformerConfig(num_layers=s["layers"], hidden_size=s["width"], num_attention_heads=s["heads"], kv_channels=s["dim"],
                            num_query_groups=max(1, s["heads"] // 4), ffn_hidden_size=s["ff"], normalization="RMSNorm",
                            add_bias_linear=False, activation_func=squared_relu, hidden_dropout=0.0, attention_dropout=0.0,
                            params_dtype=torch.bfloat16, bf16=True, num_moe_experts=s["experts"], moe_router_topk=s["top"],
                            moe_ffn_hidden_size=s["expert_ff"], moe_shared_expert_intermediate_size=s["shared_ff"],
                            moe_grouped_gemm=True, moe_token_dispatcher_type="allgather", moe_router_load_balancing_type="none",
                            moe_layer_freq=[0 if i % 4 == 0 else 1 for i in range(s["layers"])], bias_activation_fusion=False)
    model = GPTModel(cfg, get_gpt_decoder_block_spec(cfg, use_transformer_engine=False), s["vocab"], 8192,
                     position_embedding_type="rope", parallel_output=False)
    return model.to(device).eval()


def lerorax_config(s):
    """A Lerorax stack at the sizes of ``s``: side-by-side (head-mixing attention + delta memory) and minGRU layers in turn,
    every fourth layer running the weights of the layer four below, clamped gated feed-forwards of the dense size's parameter
    count."""
    ff = {"kind": "dense", "ff": s["ff"] * 2 // 3 // 64 * 64, "limit": 7.0}
    left = {"heads": s["heads"], "kv_heads": max(1, s["heads"] // 4), "dim": s["dim"], "vdim": s["dim"], "conv": 4,
            "scale": s["dim"] ** -0.5, "rot": {"base": 500000.0, "dims": s["dim"] // 2,
                                               "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 8192}}}
    right = {"heads": s["heads"], "dim": 64}
    layers = []
    for i in range(s["layers"]):
        l = {"type": "parallel", "mixer": {"left": left, "right": right}, "mlp": ff} if i % 2 == 0 else \
            {"type": "mingru", "mixer": {"width": 2 * s["width"]}, "mlp": ff}
        if i >= 4 and i % 4 in (2, 3):
            l = dict(l, weights_of=i - 4)
        layers.append(l)
    return {"architecture": "Lerorax", "vocab": s["vocab"], "width": s["width"], "norm": {"eps": 1e-5},
            "embedding": {"bigram": {"buckets": 65521, "mul_prev": 31, "mul_cur": 17}}, "layers": layers}


def build_lerorax(s, device):
    from .models.lerorax import LeroraxConfig, LeroraxModel
    from .parallel import state as ps

    if not ps.model_parallel_is_initialized():
        ps.initialize_model_parallel(1, 1)
    lcfg = LeroraxConfig.from_dict(lerorax_config(s))
    base = lcfg.base_transformer_config(torch.bfloat16, use_cpu_initialization=False)
    return LeroraxModel(lcfg, base).to(device).eval()


def domasun_config(s):
    """A Domasun stack at the sizes of ``s``: six layers of which the third to the fifth run twice in a row (eight runs), four
    residual streams, sliding-window attention (a window of 1024) beside a selective scan of twice the width with 16 states, a
    mixture of clamped gated experts with a gated shared expert."""
    left = {"heads": s["heads"], "kv_heads": max(1, s["heads"] // 4), "dim": s["dim"], "vdim": s["dim"], "scale": s["dim"] ** -0.5,
            "mask": {"size": 1024}}
    right = {"inner": 2 * s["width"], "state": 16, "dt_rank": max(8, s["width"] // 16), "conv": 4}
    moe = {"kind": "moe", "expert": {"ff": s["expert_ff"], "limit": 7.0}, "router": {"experts": s["experts"], "top": s["top"]},
           "shared": {"ff": s["shared_ff"], "limit": 7.0}}
    n = s["layers"]
    owned = n - 2 if n >= 6 else n
    layers = [{"type": "parallel", "mixer": {"left": left, "right": right, "left_scale": 0.8, "right_scale": 1.1}, "mlp": moe}
              for _ in range(owned)]
    cfg = {"architecture": "Domasun", "vocab": s["vocab"], "width": s["width"], "norm": {"eps": 1e-5}, "streams": 4,
           "logit_softcap": 30.0, "layers": layers}
    if owned < n:
        cfg["loop"] = {"start": 2, "stop": 4, "times": 2}
    return cfg


def build_domasun(s, device):
    from .models.domasun import DomasunConfig, DomasunModel
    from .parallel import state as ps

    if not ps.model_parallel_is_initialized():
        ps.initialize_model_parallel(1, 1)
    dcfg = DomasunConfig.from_dict(domasun_config(s))
    base = dcfg.base_transformer_config(torch.bfloat16, use_cpu_initialization=False)
    return DomasunModel(dcfg, base).to(device).eval()


def nunosun_config(s):
    """A Nunosun stack at the sizes of ``s``: gated delta-rule layers with a dense PolyNorm feed-forward in turn with layers of
    sliding-window attention (a window of 1024, 32 distance buckets) beside a retention memory and a mixture of SiLU-gated
    experts; a three-tap convolution in front of every mixer and a per-layer token vector of 64 numbers."""
    H, d = s["heads"], s["dim"]
    left = {"heads": H, "kv_heads": max(1, H // 4), "dim": d, "vdim": d, "scale": d ** -0.5, "mask": {"size": 1024}, "bias_max": 1024,
            "bias_buckets": 32}
    right = {"heads": H, "dim": 64, "vdim": d, "decay": [1.0 - 2.0 ** (-5 - 3.0 * h / max(1, H - 1)) for h in range(H)],
             "rot": {"dims": 64, "base": 10000.0}}
    moe = {"kind": "moe", "expert": {"ff": s["expert_ff"]}, "router": {"experts": s["experts"], "top": s["top"]}}
    dense = {"kind": "dense", "ff": s["ff"]}
    delta = {"heads": H, "kv_heads": max(1, H // 2), "dim": 64, "vdim": d, "conv": 4}
    layers = [{"type": "delta", "mixer": delta, "mlp": dense} if i % 2 == 0 else
              {"type": "parallel", "mixer": {"left": left, "right": right}, "mlp": moe} for i in range(s["layers"])]
    return {"architecture": "Nunosun", "vocab": s["vocab"], "width": s["width"], "norm": {"eps": 1e-6}, "canon": {"taps": 3},
            "token_side": {"dim": 64}, "logit_scale": 0.5, "layers": layers}


def build_nunosun(s, device):
    from .models.nunosun import NunosunConfig, NunosunModel
    from .parallel import state as ps

    if not ps.model_parallel_is_initialized():
        ps.initialize_model_parallel(1, 1)
    ncfg = NunosunConfig.from_dict(nunosun_config(s))
    base = ncfg.base_transformer_config(torch.bfloat16, use_cpu_initialization=False)
    return NunosunModel(ncfg, base).to(device).eval()


def _engine(model, max_tokens, max_requests):
    from .data.tokenizer import NullTokenizer
    from .inference import DynamicInferenceEngine

    bs = 16
    return DynamicInferenceEngine(model, NullTokenizer(1000), max_sequence_length=8192, num_blocks=max_tokens // bs + max_requests,
                                  block_size=bs, max_tokens_per_step=max_tokens, max_requests=max_requests)


def _timed(fn, steps, warmup):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(steps):
        fn()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) / steps


def serve_numbers(model, vocab, prompts, prompt_len, decoders, context, steps, warmup):
    """(prefill tokens/s, decode tokens/s) through the engine's forward."""
    g = torch.Generator().manual_seed(0)
    eng = _engine(model, max(prompts * prompt_len, decoders * (context + steps + warmup + 2)) + 64, max(prompts, decoders))
    ctx = eng.context
    n = [0]

    def prefill():
        ids = [f"p{n[0]}_{i}" for i in range(prompts)]
        n[0] += 1
        for r in ids:
            ctx.add_request(r)
        eng.forward_tokens([(r, torch.randint(0, vocab, (prompt_len,), generator=g).tolist()) for r in ids])
        for r in ids:
            ctx.release(r)

    ms_prefill = _timed(prefill, steps, warmup)
    ids = [f"d{i}" for i in range(decoders)]
    for r in ids:
        ctx.add_request(r)
    for lo in range(0, decoders, 8):                 # fill the caches
        eng.forward_tokens([(r, torch.randint(0, vocab, (context,), generator=g).tolist()) for r in ids[lo:lo + 8]])
    tok = torch.randint(0, vocab, (decoders,), generator=g).tolist()
    ms_decode = _timed(lambda: eng.forward_tokens([(r, [t]) for r, t in zip(ids, tok)]), steps, warmup)
    for r in ids:
        ctx.release(r)
    return prompts * prompt_len / ms_prefill * 1e3, decoders / ms_decode * 1e3, ms_prefill, ms_decode


def _kernel_bench(device):
    """``(bench, out, roofline)``: ``bench(name, fn, bytes, flops, like)`` times ``fn`` alone (median of 5, an L2-sized buffer
    rewritten before each) and records achieved rates and the fraction of the roofline in ``out``."""
    hbm, how = _peaks()
    fma_peak = 148 * 128 * 2 * 1.965e9 / 1e12        # fp32 TFLOP/s of the CUDA cores at the maximum clock
    flush = torch.empty(160 << 20, dtype=torch.uint8, device=device)
    out = {}

    def bench(name, fn, nbytes, flops=0.0, like=None):
        for _ in range(3):
            fn()
        ts = []
        for _ in range(5):
            flush.zero_()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            fn()
            b.record()
            torch.cuda.synchronize()
            ts.append(a.elapsed_time(b))
        ms = sorted(ts)[len(ts) // 2]
        gbs = nbytes / ms / 1e6
        tfl = flops / ms / 1e9
        frac = max(gbs / hbm, tfl / fma_peak if flops else 0.0)
        out[name] = {"ms": round(ms, 4), "GB/s": round(gbs, 1), "TFLOP/s": round(tfl, 2), "roofline_frac": round(frac, 3),
                     "bound": "fma" if flops and tfl / fma_peak > gbs / hbm else "hbm", "like": like}

    return bench, out, {"hbm_gbs": hbm, "fp32_fma_tflops": round(fma_peak, 1), "peaks": how}


def kernel_numbers_lerorax(s, device):
    """The kernels of the Lerorax mixers alone, each beside the like kernel of the closest model (Zikunex)."""
    from . import ops
    from .ops import seqmix

    bench, out, roof = _kernel_bench(device)
    H, d, W = s["heads"], s["dim"], s["width"]
    G = max(1, H // 4)
    bf = torch.bfloat16
    rn = lambda *sh, **kw: torch.randn(*sh, device=device, **kw)  # noqa: E731
    # -- decode attention: 64 requests x 2048 cached tokens; prefill: one prompt of 2048 tokens
    R, L, bs = 64, 2048, 16
    nblk = R * L // bs
    table = torch.randperm(nblk, device=device).to(torch.int32).view(R, L // bs)
    req = torch.arange(R, dtype=torch.int32, device=device)
    lens = torch.full((R,), L, dtype=torch.int32, device=device)
    kc, vc = rn(nblk * bs, G, d, dtype=bf), rn(nblk * bs, G, d, dtype=bf)
    talk = rn(H, H) * 0.3
    q = rn(R, H, d, dtype=bf)
    gate = rn(R, H * d, dtype=bf)
    bench("mixed_attention_paged.decode", lambda: seqmix.mixed_attention_paged(q, kc, vc, table, req, lens, bs, d ** -0.5, talk, gate, L),
          R * L * G * d * 2 * 2, flops=R * L * H * d * 4, like="latent_attention_paged.decode")
    r = s["kv_rank"]
    cache = rn(nblk * bs, r, dtype=bf)
    q_lat = rn(R, H, r, dtype=bf)
    bench("latent_attention_paged.decode", lambda: seqmix.latent_attention_paged(q_lat, cache, table, req, lens, bs, 0.05, L),
          R * L * r * 2, flops=R * L * H * r * 4)
    T = 2048
    table1 = torch.randperm(T // bs, device=device).to(torch.int32).view(1, -1)
    req1 = torch.zeros(T, dtype=torch.int32, device=device)
    len1 = torch.arange(1, T + 1, dtype=torch.int32, device=device)
    q1, gate1 = rn(T, H, d, dtype=bf), rn(T, H * d, dtype=bf)
    bench("mixed_attention_paged.prefill", lambda: seqmix.mixed_attention_paged(q1, kc, vc, table1, req1, len1, bs, d ** -0.5, talk, gate1, T),
          T * G * d * 4 + T * H * d * 6, flops=T * (T + 1) / 2 * H * d * 4, like="latent_attention_paged.prefill")
    q1l = rn(T, H, r, dtype=bf)
    bench("latent_attention_paged.prefill", lambda: seqmix.latent_attention_paged(q1l, cache, table1, req1, len1, bs, 0.05, T),
          T * r * 2 + T * H * r * 6, flops=T * (T + 1) / 2 * H * r * 4)
    # -- matrix-memory scans: decode (64 sequences x 1 token, state bound) and prefill (4 x 2048 tokens, FMA bound); key dim 64
    dd = 64
    for tag, R_, n in (("decode", 64, 1), ("prefill", 4, 2048)):
        T_ = R_ * n
        pb = seqmix.PackedBatch([i * n for i in range(R_ + 1)], list(range(R_)), device)
        rr, k, v = rn(T_, H, dd, dtype=bf), rn(T_, H, dd, dtype=bf), rn(T_, H, dd, dtype=bf)
        wp, ap, wb = rn(T_, H * dd, dtype=bf), rn(T_, H * dd, dtype=bf), rn(H * dd, dtype=bf)
        S = torch.zeros(R_, H, dd, dd, device=device)
        state_bytes = R_ * H * dd * dd * 4 * 2
        io = T_ * H * dd * 2 * 5 + T_ * H * dd * 4
        bench(f"gen_delta_scan.{tag}", lambda: seqmix.gen_delta_scan(rr, k, v, wp, ap, wb, pb, S, 0.6), state_bytes + io,
              flops=T_ * H * dd * dd * 10, like=f"delta_rule_scan.{tag}")
        ld = -torch.rand(T_, H, dd, device=device) * 0.1
        beta = torch.rand(T_, H, device=device)
        bench(f"delta_rule_scan.{tag}", lambda: seqmix.delta_rule_scan(rr, k, v, ld, beta, pb, S),
              state_bytes + T_ * H * dd * 2 * 3 + T_ * H * dd * 4 * 2, flops=T_ * H * dd * dd * 8)
        C = 2 * W
        zp, up, gp = rn(T_, C, dtype=bf), rn(T_, C, dtype=bf), rn(T_, C, dtype=bf)
        Sg = torch.zeros(R_, C, device=device)
        bench(f"mingru_scan.{tag}", lambda: seqmix.mingru_scan(zp, up, gp, pb, Sg), T_ * C * 2 * 4 + R_ * C * 8, like="add_rms_norm")
    # -- norms, convolution, gate over 8192 tokens
    T = 8192
    x = rn(T, W)
    a, b = rn(T, W, dtype=bf), rn(T, W, dtype=bf)
    w = torch.ones(W, device=device, dtype=bf)
    bench("norm_add", lambda: seqmix.norm_add(x, a, w, 1e-5, bf, 1.0), T * W * (4 + 4 + 2 + 2), like="add_rms_norm")
    bench("norm_add (two branches)", lambda: seqmix.norm_add(x, a, w, 1e-5, bf, 1.0, b, w, w), T * W * (4 + 4 + 2 + 2 + 2), like="add_rms_norm")
    bench("add_rms_norm", lambda: seqmix.add_rms_norm(x, a, w, 1e-5, bf), T * W * (4 + 4 + 2 + 2))
    qk = rn(T, (H + 2 * G) * d, dtype=bf)
    wq, wk = torch.ones(H * d, device=device, dtype=bf), torch.ones(G * d, device=device, dtype=bf)
    pos = torch.arange(T, device=device)
    inv = torch.rand(d // 4, device=device)
    bench("norm_rope", lambda: seqmix.norm_rope(qk[:, :H * d], qk[:, H * d:(H + G) * d], wq, wk, pos, inv, d, d // 2, 1e-5),
          T * (H + G) * d * 4, like="add_rms_norm")
    C = (H + 2 * G) * d
    wc = rn(C, 4, dtype=bf)
    pbc = seqmix.PackedBatch([0, T], [0], device)
    win = torch.zeros(1, 3, C, device=device, dtype=bf)
    bench("causal_conv", lambda: seqmix.causal_conv(qk, wc, pbc, win), T * C * 4, like="causal_conv_silu")
    bench("causal_conv_silu", lambda: seqmix.causal_conv_silu(qk, wc, pbc, win), T * C * 4)
    F_ = s["ff"] * 2 // 3 // 64 * 64
    xf = rn(T, 2 * F_, dtype=bf)
    bench("clamped_glu", lambda: seqmix.clamped_glu(xf, 7.0), T * F_ * 6, like="swiglu")
    bench("swiglu", lambda: ops.swiglu(xf, None), T * F_ * 6)
    return out, roof


def kernel_numbers_domasun(s, device):
    """The kernels of the Domasun layers alone, each beside the like kernel of the closest model (Lerorax)."""
    from .ops import seqmix
    from .transformer.window_attention import distance_slopes

    bench, out, roof = _kernel_bench(device)
    H, d, W = s["heads"], s["dim"], s["width"]
    G = max(1, H // 4)
    bf = torch.bfloat16
    rn = lambda *sh, **kw: torch.randn(*sh, device=device, **kw)  # noqa: E731
    # -- decode attention: 64 requests x 2048 cached tokens of which a window of 1024 is visible; prefill: one prompt of 2048
    R, L, bs, win = 64, 2048, 16, 1024
    nblk = R * L // bs
    table = torch.randperm(nblk, device=device).to(torch.int32).view(R, L // bs)
    req = torch.arange(R, dtype=torch.int32, device=device)
    lens = torch.full((R,), L, dtype=torch.int32, device=device)
    kc, vc = rn(nblk * bs, G, d, dtype=bf), rn(nblk * bs, G, d, dtype=bf)
    slopes = distance_slopes(H).to(device)
    q, gate = rn(R, H, d, dtype=bf), rn(R, H, dtype=bf)
    bench("window_attention_paged.decode", lambda: seqmix.window_attention_paged(q, kc, vc, table, req, lens, bs, d ** -0.5, win, slopes,
                                                                                 True, gate, 1.0, L),
          R * win * G * d * 2 * 2, flops=R * win * H * d * 4, like="mixed_attention_paged.decode")
    talk = rn(H, H) * 0.3
    gate_m = rn(R, H * d, dtype=bf)
    bench("mixed_attention_paged.decode", lambda: seqmix.mixed_attention_paged(q, kc, vc, table, req, lens, bs, d ** -0.5, talk, gate_m, L),
          R * L * G * d * 2 * 2, flops=R * L * H * d * 4)
    T = 2048
    table1 = torch.randperm(T // bs, device=device).to(torch.int32).view(1, -1)
    req1 = torch.zeros(T, dtype=torch.int32, device=device)
    len1 = torch.arange(1, T + 1, dtype=torch.int32, device=device)
    q1, gate1, gate1m = rn(T, H, d, dtype=bf), rn(T, H, dtype=bf), rn(T, H * d, dtype=bf)
    pairs = win * (win + 1) / 2 + (T - win) * win                     # visible (query, key) pairs under the window
    bench("window_attention_paged.prefill", lambda: seqmix.window_attention_paged(q1, kc, vc, table1, req1, len1, bs, d ** -0.5, win,
                                                                                  slopes, True, gate1),
          T * G * d * 4 + T * H * d * 4, flops=pairs * H * d * 4, like="mixed_attention_paged.prefill")
    bench("mixed_attention_paged.prefill", lambda: seqmix.mixed_attention_paged(q1, kc, vc, table1, req1, len1, bs, d ** -0.5, talk, gate1m, T),
          T * G * d * 4 + T * H * d * 6, flops=T * (T + 1) / 2 * H * d * 4)
    # -- scans: decode (64 sequences x 1 token, state bound) and prefill (4 x 2048 tokens)
    C, N = 2 * W, 16
    dd = 64
    for tag, R_, n in (("decode", 64, 1), ("prefill", 4, 2048)):
        T_ = R_ * n
        pb = seqmix.PackedBatch([i * n for i in range(R_ + 1)], list(range(R_)), device)
        x, z, B, Cm = rn(T_, C, dtype=bf), rn(T_, C, dtype=bf), rn(T_, N, dtype=bf), rn(T_, N, dtype=bf)
        dtp = rn(T_, C) - 2.0
        A_log, D, dtb = (torch.rand(C, N, device=device) + 0.1).log().to(bf), rn(C, dtype=bf), rn(C, dtype=bf)
        S = torch.zeros(R_, C, N, device=device)
        bench(f"selective_scan.{tag}", lambda: seqmix.selective_scan(x, dtp, B, Cm, A_log, D, pb, S, z, dtb),
              R_ * C * N * 8 + T_ * C * (2 + 2 + 4 + 2) + C * N * 2, flops=T_ * C * N * 6, like=f"gen_delta_scan.{tag}")
        rr, k, v = rn(T_, H, dd, dtype=bf), rn(T_, H, dd, dtype=bf), rn(T_, H, dd, dtype=bf)
        wp, ap, wb = rn(T_, H * dd, dtype=bf), rn(T_, H * dd, dtype=bf), rn(H * dd, dtype=bf)
        Sd = torch.zeros(R_, H, dd, dd, device=device)
        bench(f"gen_delta_scan.{tag}", lambda: seqmix.gen_delta_scan(rr, k, v, wp, ap, wb, pb, Sd, 0.6),
              R_ * H * dd * dd * 8 + T_ * H * dd * 2 * 5 + T_ * H * dd * 4, flops=T_ * H * dd * dd * 10)
    # -- stream update + norm, per-head norm, positions, convolution over 8192 tokens
    T, S_ = 8192, 4
    X = rn(T, S_, W)
    a, b = rn(T, W, dtype=bf), rn(T, W, dtype=bf)
    w = torch.ones(W, device=device, dtype=bf)
    mix, outc, inp = torch.eye(S_, device=device), torch.ones(S_, device=device), torch.full((S_,), 0.25, device=device)
    bench("stream_mix_norm (4 streams, two branches)",
          lambda: seqmix.stream_mix_norm(X, a, b, w, w, 0.8, 1.1, mix, outc, inp, w, w, 1e-5), T * W * (S_ * 8 + 2 + 2 + 2),
          like="norm_add (two branches)")
    X1 = rn(T, 1, W)
    bench("stream_mix_norm (1 stream)", lambda: seqmix.stream_mix_norm(X1, a, None, None, w, 1.0, 1.0, mix[:1, :1].contiguous(), outc[:1],
                                                                      outc[:1], w, w, 1e-5), T * W * (8 + 2 + 2), like="add_rms_norm")
    x = rn(T, W)
    bench("norm_add (two branches)", lambda: seqmix.norm_add(x, a, w, 1e-5, bf, 1.0, b, w, w), T * W * (4 + 4 + 2 + 2 + 2))
    bench("add_rms_norm", lambda: seqmix.add_rms_norm(x, a, w, 1e-5, bf), T * W * (4 + 4 + 2 + 2))
    qk = rn(T, (H + G) * d + H, dtype=bf)
    wn = torch.ones(d, device=device, dtype=bf)
    bench("head_rms_norm (q and k)", lambda: (seqmix.head_rms_norm(qk[:, :H * d].view(T, H, d), wn, 1e-5),
                                             seqmix.head_rms_norm(qk[:, H * d:(H + G) * d].view(T, G, d), wn, 1e-5)),
          T * (H + G) * d * 4, like="norm_rope")
    wq, wk = torch.ones(H * d, device=device, dtype=bf), torch.ones(G * d, device=device, dtype=bf)
    pos = torch.arange(T, device=device)
    inv = torch.rand(d // 4, device=device)
    bench("norm_rope", lambda: seqmix.norm_rope(qk[:, :H * d], qk[:, H * d:(H + G) * d], wq, wk, pos, inv, d, d // 2, 1e-5),
          T * (H + G) * d * 4)
    freq = torch.rand(W // 2, device=device)
    bench("add_sinusoid", lambda: seqmix.add_sinusoid(x, pos, freq), T * W * 8, like="add_rms_norm")
    xc, wc, cb = rn(T, C, dtype=bf), rn(C, 4, dtype=bf), rn(C, dtype=bf)
    pbc = seqmix.PackedBatch([0, T], [0], device)
    winc = torch.zeros(1, 3, C, device=device, dtype=bf)
    bench("causal_conv_silu (bias)", lambda: seqmix.causal_conv_silu(xc, wc, pbc, winc, cb), T * C * 4, like="causal_conv_silu")
    bench("causal_conv_silu", lambda: seqmix.causal_conv_silu(xc, wc, pbc, winc), T * C * 4)
    return out, roof


def kernel_numbers_nunosun(s, device):
    """The kernels of the Nunosun layers alone, each beside the like kernel of the closest models (Domasun, Zikunex)."""
    from .ops import seqmix
    from .transformer.window_attention import distance_buckets, distance_slopes

    bench, out, roof = _kernel_bench(device)
    H, d, W = s["heads"], s["dim"], s["width"]
    G = max(1, H // 4)
    bf = torch.bfloat16
    rn = lambda *sh, **kw: torch.randn(*sh, device=device, **kw)  # noqa: E731
    # -- decode attention: 64 requests x 2048 cached tokens of which a window of 1024 is visible; prefill: one prompt of 2048
    R, L, bs, win = 64, 2048, 16, 1024
    nblk = R * L // bs
    table = torch.randperm(nblk, device=device).to(torch.int32).view(R, L // bs)
    req = torch.arange(R, dtype=torch.int32, device=device)
    lens = torch.full((R,), L, dtype=torch.int32, device=device)
    kc, vc = rn(nblk * bs, G, d, dtype=bf), rn(nblk * bs, G, d, dtype=bf)
    slopes = distance_slopes(H).to(device)
    bias = rn(32, H)[distance_buckets(32, 1024.0, win).to(device)].contiguous()
    q, gate = rn(R, H, d, dtype=bf), rn(R, H, dtype=bf)
    bench("window_attention_paged.decode (distance bias)",
          lambda: seqmix.window_attention_paged(q, kc, vc, table, req, lens, bs, d ** -0.5, win, None, False, None, 1.0, L, bias),
          R * win * G * d * 2 * 2, flops=R * win * H * d * 4, like="window_attention_paged.decode (slopes, sink, gate)")
    bench("window_attention_paged.decode (slopes, sink, gate)",
          lambda: seqmix.window_attention_paged(q, kc, vc, table, req, lens, bs, d ** -0.5, win, slopes, True, gate, 1.0, L),
          R * win * G * d * 2 * 2, flops=R * win * H * d * 4)
    T = 2048
    table1 = torch.randperm(T // bs, device=device).to(torch.int32).view(1, -1)
    req1 = torch.zeros(T, dtype=torch.int32, device=device)
    len1 = torch.arange(1, T + 1, dtype=torch.int32, device=device)
    q1, gate1 = rn(T, H, d, dtype=bf), rn(T, H, dtype=bf)
    pairs = win * (win + 1) / 2 + (T - win) * win                     # visible (query, key) pairs under the window
    bench("window_attention_paged.prefill (distance bias)",
          lambda: seqmix.window_attention_paged(q1, kc, vc, table1, req1, len1, bs, d ** -0.5, win, None, False, None, 1.0, 0, bias),
          T * G * d * 4 + T * H * d * 4, flops=pairs * H * d * 4, like="window_attention_paged.prefill (slopes, sink, gate)")
    bench("window_attention_paged.prefill (slopes, sink, gate)",
          lambda: seqmix.window_attention_paged(q1, kc, vc, table1, req1, len1, bs, d ** -0.5, win, slopes, True, gate1),
          T * G * d * 4 + T * H * d * 4, flops=pairs * H * d * 4)
    # -- matrix memories: decode (64 sequences x 1 token, state bound) and prefill (4 x 2048 tokens, FMA bound); key dim 64
    dd = 64
    for tag, R_, n in (("decode", 64, 1), ("prefill", 4, 2048)):
        T_ = R_ * n
        pb = seqmix.PackedBatch([i * n for i in range(R_ + 1)], list(range(R_)), device)
        qq, k, v = rn(T_, H, dd, dtype=bf), rn(T_, H, dd, dtype=bf), rn(T_, H, d, dtype=bf)
        S = torch.zeros(R_, H, dd, d, device=device)
        state_bytes = R_ * H * dd * d * 4 * 2
        decay = torch.rand(H, device=device) * 0.05 + 0.95
        pos = torch.arange(n, device=device).repeat(R_) + (1024 if n == 1 else 0)
        inv = seqmix.rotary_frequencies(dd, 10000.0, device)
        bench(f"retention_scan.{tag}", lambda: seqmix.retention_scan(qq, k, v, decay, pb, S, pos, inv, dd ** -0.5),
              state_bytes + T_ * H * (2 * dd + d) * 2 + T_ * H * d * 4, flops=T_ * H * dd * d * 4, like=f"delta_rule_scan.{tag} (decay per channel)")
        ldc = -torch.rand(T_, H, dd, device=device) * 0.1
        ldh = -torch.rand(T_, H, device=device) * 0.1
        beta = torch.rand(T_, H, device=device)
        kq, kk = rn(T_, H // 2, dd, dtype=bf), rn(T_, H // 2, dd, dtype=bf)
        io = T_ * (H // 2) * dd * 2 * 2 + T_ * H * d * 2 + T_ * H * d * 4
        bench(f"delta_rule_scan.{tag} (decay per head)", lambda: seqmix.delta_rule_scan(kq, kk, v, ldh, beta, pb, S, 1e-6, dd ** -0.5),
              state_bytes + io + T_ * H * 8, flops=T_ * H * dd * d * 8, like=f"delta_rule_scan.{tag} (decay per channel)")
        bench(f"delta_rule_scan.{tag} (decay per channel)", lambda: seqmix.delta_rule_scan(kq, kk, v, ldc, beta, pb, S, 1e-6, dd ** -0.5),
              state_bytes + io + T_ * H * (dd + 1) * 4, flops=T_ * H * dd * d * 8)
    # -- additions and norms, convolution, activations over 8192 tokens
    T = 8192
    x = rn(T, W)
    a, b, f = rn(T, W, dtype=bf), rn(T, W, dtype=bf), rn(T, W, dtype=bf)
    w = torch.ones(W, device=device, dtype=bf)
    bench("norm_add (two branches + feed-forward, no outer norm)", lambda: seqmix.norm_add(x, a, None, 1e-6, bf, 0.0, b, w, w, extra=f),
          T * W * (4 + 4 + 2 + 2 + 2 + 2), like="norm_add (two branches)")
    bench("norm_add (normed addend + next norm)", lambda: seqmix.norm_add(x, a, w, 1e-6, bf, next_weight=w), T * W * (4 + 4 + 2 + 2),
          like="norm_add (two branches)")
    bench("norm_add (two branches)", lambda: seqmix.norm_add(x, a, w, 1e-5, bf, 1.0, b, w, w), T * W * (4 + 4 + 2 + 2 + 2))
    bench("add_rms_norm", lambda: seqmix.add_rms_norm(x, a, w, 1e-5, bf), T * W * (4 + 4 + 2 + 2))
    o = rn(T, H, d)
    gt = rn(T, H * d, dtype=bf)
    wn = torch.ones(d, device=device, dtype=bf)
    bench("gated_head_rms_norm (no weight, silu gate)", lambda: seqmix.gated_head_rms_norm(o, None, gt, 1e-6, bf, "silu"), T * H * d * (4 + 2 + 2),
          like="gated_head_rms_norm (weight, sigmoid gate)")
    bench("gated_head_rms_norm (weight, sigmoid gate)", lambda: seqmix.gated_head_rms_norm(o, wn, gt, 1e-6, bf), T * H * d * (4 + 2 + 2))
    h = rn(T, W, dtype=bf)
    wc3 = rn(W, 3, dtype=bf)
    pbc = seqmix.PackedBatch([0, T], [0], device)
    win3 = torch.zeros(1, 2, W, device=device, dtype=bf)
    bench("causal_conv (3 taps, input added)", lambda: seqmix.causal_conv(h, wc3, pbc, win3, residual=True), T * W * 4, like="causal_conv_silu")
    C = (H + H // 2 * 2) * 64
    xc, wc = rn(T, C, dtype=bf), rn(C, 4, dtype=bf)
    winc = torch.zeros(1, 3, C, device=device, dtype=bf)
    bench("causal_conv_silu", lambda: seqmix.causal_conv_silu(xc, wc, pbc, winc), T * C * 4)
    F_ = s["ff"]
    z = rn(T, F_, dtype=bf)
    coef = torch.tensor([0.8, 0.3, -0.2, 0.1], device=device)
    bench("poly_norm", lambda: seqmix.poly_norm(z, coef, 1e-6), T * F_ * 4, like="clamped_glu")
    z2 = rn(T, 2 * F_, dtype=bf)
    bench("clamped_glu", lambda: seqmix.clamped_glu(z2, 7.0), T * F_ * 6)
    g64, e64 = rn(T, 64, dtype=bf), rn(T, 64 * s["layers"], dtype=bf)
    bench("gelu_mul", lambda: seqmix.gelu_mul(g64, e64[:, 64:128]), T * 64 * 6, like="clamped_glu")
    return out, roof


def kernel_numbers(s, device):
    """Every new kernel alone and its like kernel: time, achieved bytes/s (or flop/s) and the fraction of the roofline."""
    from . import ops
    from .ops import seqmix

    hbm, how = _peaks()
    fma_peak = 148 * 128 * 2 * 1.965e9 / 1e12        # fp32 TFLOP/s of the CUDA cores at the maximum clock
    flush = torch.empty(160 << 20, dtype=torch.uint8, device=device)
    out = {}

    def bench(name, fn, nbytes, flops=0.0, like=None):
        for _ in range(3):
            fn()
        ts = []
        for _ in range(5):
            flush.zero_()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            fn()
            b.record()
            torch.cuda.synchronize()
            ts.append(a.elapsed_time(b))
        ms = sorted(ts)[len(ts) // 2]
        gbs = nbytes / ms / 1e6
        tfl = flops / ms / 1e9
        frac = max(gbs / hbm, tfl / fma_peak if flops else 0.0)
        out[name] = {"ms": round(ms, 4), "GB/s": round(gbs, 1), "TFLOP/s": round(tfl, 2), "roofline_frac": round(frac, 3),
                     "bound": "fma" if flops and tfl / fma_peak > gbs / hbm else "hbm", "like": like}

    H, d, r, W = s["heads"], s["dim"], s["kv_rank"], s["width"]
    bf = torch.bfloat16
    # -- decode attention: 64 requests x 2048 cached tokens
    R, L, bs = 64, 2048, 16
    nblk = R * L // bs
    table = torch.randperm(nblk, device=device).to(torch.int32).view(R, L // bs)
    req = torch.arange(R, dtype=torch.int32, device=device)
    lens = torch.full((R,), L, dtype=torch.int32, device=device)
    cache = torch.randn(nblk * bs, r, device=device, dtype=bf)
    q_lat = torch.randn(R, H, r, device=device, dtype=bf)
    bench("latent_attention_paged.decode", lambda: seqmix.latent_attention_paged(q_lat, cache, table, req, lens, bs, 0.05, L),
          R * L * r * 2, flops=R * L * H * r * 4, like="paged_attention.decode")
    ng = max(1, H // 4)
    kc = torch.randn(nblk * bs, ng, d, device=device, dtype=bf)
    vc = torch.randn(nblk * bs, ng, d, device=device, dtype=bf)
    qg = torch.randn(R, H, d, device=device, dtype=bf)
    if ops.ext().paged_attention_supported(d, H // ng):
        bench("paged_attention.decode", lambda: ops.ext().paged_attention(qg, kc, vc, table, req, lens, bs, d ** -0.5, 1),
              R * L * ng * d * 2 * 2, flops=R * L * H * d * 4)
    # -- prefill attention: one prompt of 2048 tokens
    T = 2048
    table1 = torch.randperm(T // bs, device=device).to(torch.int32).view(1, -1)
    req1 = torch.zeros(T, dtype=torch.int32, device=device)
    len1 = torch.arange(1, T + 1, dtype=torch.int32, device=device)
    q1 = torch.randn(T, H, r, device=device, dtype=bf)
    bench("latent_attention_paged.prefill", lambda: seqmix.latent_attention_paged(q1, cache, table1, req1, len1, bs, 0.05, T),
          T * r * 2 + T * H * r * 6, flops=T * (T + 1) / 2 * H * r * 4, like="paged_attention.prefill")
    qg1 = torch.randn(T, H, d, device=device, dtype=bf)
    if ops.ext().paged_attention_supported(d, H // ng):
        bench("paged_attention.prefill", lambda: ops.ext().paged_attention(qg1, kc, vc, table1, req1, len1, bs, d ** -0.5, 1),
              T * ng * d * 4 + T * H * d * 4, flops=T * (T + 1) / 2 * H * d * 4)
    # -- scans: decode (64 sequences x 1 token, state bound) and prefill (4 x 2048 tokens, FMA bound)
    for tag, R_, n in (("decode", 64, 1), ("prefill", 4, 2048)):
        T_ = R_ * n
        pb = seqmix.PackedBatch([i * n for i in range(R_ + 1)], list(range(R_)), device)
        q = torch.randn(T_, H, d, device=device, dtype=bf)
        k = torch.randn(T_, H, d, device=device, dtype=bf)
        v = torch.randn(T_, H, d, device=device, dtype=bf)
        ld = -torch.rand(T_, H, d, device=device) * 0.1
        beta = torch.rand(T_, H, device=device)
        S = torch.zeros(R_, H, d, d, device=device)
        state_bytes = R_ * H * d * d * 4 * 2
        io = T_ * H * d * 2 * 3 + T_ * H * d * 4 * 2
        bench(f"delta_rule_scan.{tag}", lambda: seqmix.delta_rule_scan(q, k, v, ld, beta, pb, S), state_bytes + io,
              flops=T_ * H * d * d * 8, like="ssd_scan (PyTorch)")
        li, lf = torch.randn(T_, H, device=device), -torch.rand(T_, H, device=device)
        nS, mS = torch.zeros(R_, H, d, device=device), torch.zeros(R_, H, device=device)
        bench(f"mlstm_scan.{tag}", lambda: seqmix.mlstm_scan(q, k, v, li, lf, pb, S, nS, mS, d ** -0.5), state_bytes + io,
              flops=T_ * H * d * d * 4, like="ssd_scan (PyTorch)")
        from .ssm.mamba import ssd_scan

        x4 = v.view(R_, n, H, d)
        dt = torch.rand(R_, n, H, device=device) * 0.1
        A = -torch.rand(H, device=device)
        B4, C4 = k.view(R_, n, H, d)[:, :, :1], q.view(R_, n, H, d)[:, :, :1]
        Dp = torch.ones(H, device=device)
        S0 = torch.zeros(R_, H, d, d, device=device)
        bench(f"ssd_scan (PyTorch).{tag}", lambda: ssd_scan(x4, dt, A, B4, C4, Dp, 64, S0), state_bytes + io, flops=T_ * H * d * d * 4)
    # -- norms and convolution over 8192 tokens
    T = 8192
    x = torch.randn(T, W, device=device)
    delta = torch.randn(T, W, device=device, dtype=bf)
    w = torch.ones(W, device=device, dtype=bf)
    bench("add_rms_norm", lambda: seqmix.add_rms_norm(x, delta, w, 1e-5, bf), T * W * (4 + 4 + 2 + 2), like="layer_norm (rms)")
    xb = torch.randn(T, W, device=device, dtype=bf)
    bench("layer_norm (rms)", lambda: ops.layer_norm(xb, w, None, 1e-5, rms=True), T * W * 4)
    o = torch.randn(T, H, d, device=device)
    gate = torch.randn(T, H * d, device=device, dtype=bf)
    wn = torch.ones(d, device=device, dtype=bf)
    bench("gated_head_rms_norm", lambda: seqmix.gated_head_rms_norm(o, wn, gate, 1e-5, bf), T * H * d * (4 + 2 + 2), like="layer_norm (rms)")
    C = 3 * H * d
    xc = torch.randn(T, C, device=device, dtype=bf)
    wc = torch.randn(C, 4, device=device, dtype=bf)
    pbc = seqmix.PackedBatch([0, T], [0], device)
    win = torch.zeros(1, 3, C, device=device, dtype=bf)
    bench("causal_conv_silu", lambda: seqmix.causal_conv_silu(xc, wc, pbc, win), T * C * 4, like="layer_norm (rms)")
    lg = torch.randn(T, s["experts"], device=device)
    bench("group_limited_router", lambda: seqmix.group_limited_router(lg, s["top"], 4, 2), T * s["experts"] * 9, like="router_topk")
    from .ops.moe import router_topk

    bench("router_topk", lambda: router_topk(lg, s["top"], True, None), T * s["experts"] * 9)
    return out, {"hbm_gbs": hbm, "fp32_fma_tflops": round(fma_peak, 1), "peaks": how}


def run(args):
    assert torch.cuda.is_available(), "--serving needs a GPU"
    dev = "cuda:0"
    torch.cuda.set_device(0)
    s = SIZES[args.serving_size]
    res = {"metric": "serving_tokens_per_s", "size": args.serving_size, "dtype": "bf16", "data": "synthetic", "steps": args.steps,
           "warmup": max(3, args.warmup), "config": dict(s, prompts=4, prompt_len=2048, decoders=32, context=1024,
                                                        l2="model steps read weights and caches larger than L2; kernel "
                                                           "timings rewrite a 160 MB buffer between launches")}
    design = getattr(args, "serving_design", "zikunex")
    res["design"] = design
    pairs = {"zikunex": (("zikunex", build_zikunex), ("gpt_gqa_moe", build_gpt)),
             "lerorax": (("lerorax", build_lerorax), ("zikunex", build_zikunex)),
             "domasun": (("domasun", build_domasun), ("lerorax", build_lerorax)),
             "nunosun": (("nunosun", build_nunosun), ("domasun", build_domasun))}[design]
    with torch.no_grad():
        for name, build in pairs:
            t0 = time.time()
            model = build(s, dev)
            pre, dec, ms_p, ms_d = serve_numbers(model, s["vocab"], 4, 2048, 32, 1024, args.steps, max(3, args.warmup))
            res[name] = {"prefill_tokens_per_s": round(pre, 1), "decode_tokens_per_s": round(dec, 1), "prefill_ms": round(ms_p, 2),
                         "decode_ms": round(ms_d, 2), "params_M": round(sum(p.numel() for p in model.parameters()) / 1e6, 1),
                         "build_s": round(time.time() - t0, 1)}
            del model
            torch.cuda.empty_cache()
        if not getattr(args, "serving_models_only", False):
            fn = {"zikunex": kernel_numbers, "lerorax": kernel_numbers_lerorax, "domasun": kernel_numbers_domasun,
                  "nunosun": kernel_numbers_nunosun}[design]
            res["kernels"], res["roofline"] = fn(s, dev)
    print(json.dumps(res), flush=True)
    return res
