"""A plain, slow evaluation of the Domasun design, written from its equations: one function per mechanism, loops over tokens
where the design is sequential, float64 throughout.  It shares no code with the framework.

Weights are a dict of checkpoint-named tensors (``embed``, ``l<i>.mix.left.q`` ..., ``head``), linear weights ``[out, in]``.
"""
import math

import torch

F64 = torch.float64


def sinusoid(n_tokens, width, first=0):
    """Row p: entries (2i, 2i + 1) = (sin, cos)(p * 10000^(-2i / width))."""
    out = torch.zeros(n_tokens, width, dtype=F64)
    for t in range(n_tokens):
        for i in range(width // 2):
            a = (first + t) * 10000.0 ** (-2.0 * i / width)
            out[t, 2 * i], out[t, 2 * i + 1] = math.sin(a), math.cos(a)
    return out


def layer_norm(x, w, b, eps):
    mu = x.mean(-1, keepdim=True)
    var = ((x - mu) ** 2).mean(-1, keepdim=True)
    return (x - mu) / torch.sqrt(var + eps) * w + b


def head_rms(x, w, eps):
    """x [.., dim]: divided by its root mean square, times w."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * w


def slopes(heads, exponent=8.0):
    return [2.0 ** (-exponent * (h + 1) / heads) for h in range(heads)]


def window_attention(q, k, v, scale, window, slope, sink=True, first=0):
    """q [T, H, d], k [L, G, d], v [L, G, dv] with L = first + T cached positions; query t sits at position first + t and sees
    positions j with 0 <= i - j < window (window 0: all).  Returns [T, H, dv]."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros(T, H, v.shape[2], dtype=F64)
    for t in range(T):
        i = first + t
        lo = 0 if not window else max(0, i - window + 1)
        for h in range(H):
            g = h // (H // G)
            s = torch.stack([(q[t, h] * k[j, g]).sum() * scale - slope[h] * (i - j) for j in range(lo, i + 1)])
            e = torch.exp(s)
            p = e / ((1.0 if sink else 0.0) + e.sum())
            for n, j in enumerate(range(lo, i + 1)):
                out[t, h] += p[n] * v[j, g]
    return out


def left_mixer(x, W, p, c, eps):
    H, G, d = c["heads"], c.get("kv_heads", c["heads"]), c["dim"]
    T = x.shape[0]
    q = (x @ W[p + "q"].T + W[p + "q.b"]).view(T, H, d)
    k = (x @ W[p + "k"].T + W[p + "k.b"]).view(T, G, d)
    o = window_attention(head_rms(q, W[p + "q.norm"], eps), head_rms(k, W[p + "k.norm"], eps), k, c["scale"],
                         (c.get("mask") or {}).get("size", 0), slopes(H))
    o = o * torch.sigmoid(x @ W[p + "g"].T).unsqueeze(-1)
    return o.reshape(T, H * d) @ W[p + "o"].T + W[p + "o.b"]


def causal_conv(u, w, b):
    """y_t = b + sum_j w[:, j] u_(t - taps + 1 + j), zeros before the start."""
    T, taps = u.shape[0], w.shape[1]
    y = torch.zeros_like(u)
    for t in range(T):
        y[t] = b
        for j in range(taps):
            s = t - taps + 1 + j
            if s >= 0:
                y[t] = y[t] + w[:, j] * u[s]
    return y


def silu(x):
    return x * torch.sigmoid(x)


def selective_scan(x, dt, A, B, C, D):
    """x, dt [T, C]; A [C, N]; B, C [T, N]."""
    S = torch.zeros_like(A)
    ys = []
    for t in range(x.shape[0]):
        S = torch.exp(dt[t].unsqueeze(1) * A) * S + (dt[t] * x[t]).unsqueeze(1) * B[t].unsqueeze(0)
        ys.append((S * C[t].unsqueeze(0)).sum(1) + D * x[t])
    return torch.stack(ys)


def right_mixer(h, W, p, c):
    inner, N, R = c["inner"], c["state"], c["dt_rank"]
    xz = h @ W[p + "in"].T
    x, z = xz[:, :inner], xz[:, inner:]
    x = silu(causal_conv(x, W[p + "conv"], W[p + "conv.b"]))
    low = x @ W[p + "x"].T
    dt = torch.log1p(torch.exp(low[:, :R] @ W[p + "dt"].T + W[p + "dt.b"]))
    y = selective_scan(x, dt, -torch.exp(W[p + "A_log"]), low[:, R:R + N], low[:, R + N:], W[p + "D"])
    return (y * silu(z)) @ W[p + "o"].T


def expert(h, W, p, limit):
    g = torch.clamp(h @ W[p + "gate"].T, max=limit)
    u = torch.clamp(h @ W[p + "up"].T, -limit, limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ W[p + "down"].T


def route(z, top):
    """Router logits [E] -> [(expert, weight)]: the ``top`` largest, softmax over those alone."""
    order = sorted(range(len(z)), key=lambda e: -float(z[e]))[:top]
    w = torch.softmax(torch.stack([z[e] for e in order]), 0)
    return [(e, w[n]) for n, e in enumerate(order)]


def mixture(h, W, p, c):
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, w in route(h[t] @ W[p + "router"].T, c["router"]["top"]):
            out[t] += w * expert(h[t:t + 1], W, f"{p}e{e}.", c["expert"]["limit"])[0]
    if c.get("shared"):
        out = out + torch.sigmoid(h @ W[p + "shared.sg"].T) * expert(h, W, p + "shared.", c["shared"]["limit"])
    return out


def runs_of(cfg):
    n, lp = len(cfg["layers"]), cfg.get("loop")
    if not lp:
        return list(range(n))
    return list(range(lp["start"])) + list(range(lp["start"], lp["stop"])) * lp["times"] + list(range(lp["stop"], n))


def forward(cfg, W, tokens, return_layers=False):
    """Logits [T, vocab] of one sequence (and the sum of the streams after every layer run)."""
    W = {k: v.to(F64) for k, v in W.items()}
    eps, width = cfg["norm"]["eps"], cfg["width"]
    x = W["embed"][torch.tensor(tokens)] + sinusoid(len(tokens), width)
    hyper = cfg.get("streams") is not None
    S = cfg["streams"] if hyper else 1
    xs = [x.clone() for _ in range(S)]
    seen = []
    for i in runs_of(cfg):
        L, p = cfg["layers"][i], f"l{i}."
        for q in (1, 2):
            if q == 2 and not L.get("mlp"):
                continue
            if hyper:
                w_in, w_out, w_mix = W[f"{p}hc{q}.in"], W[f"{p}hc{q}.out"], W[f"{p}hc{q}.mix"]
            else:
                w_in, w_out, w_mix = torch.ones(1, dtype=F64), torch.ones(1, dtype=F64), torch.ones(1, 1, dtype=F64)
            u = sum(w_in[s] * xs[s] for s in range(S))
            h = layer_norm(u, W[f"{p}norm{q}"], W[f"{p}norm{q}.b"], eps)
            if q == 1:
                m = L["mixer"]
                y = m["left_scale"] * left_mixer(h, W, p + "mix.left.", m["left"], eps) + \
                    m["right_scale"] * right_mixer(h, W, p + "mix.right.", m["right"])
            else:
                y = mixture(h, W, p + "mlp.", L["mlp"])
            y = y * W[f"{p}ls{q}"]
            xs = [sum(w_mix[s, t] * xs[s] for s in range(S)) + w_out[t] * y for t in range(S)]
        seen.append(sum(xs))
    logits = layer_norm(sum(xs), W["final.norm"], W["final.norm.b"], eps) @ W["head"].T
    cap = cfg.get("logit_softcap")
    if cap:
        logits = cap * torch.tanh(logits / cap)
    return (logits, seen) if return_layers else logits


def random_weights(cfg, seed=0, dtype=torch.float32):
    """Checkpoint-named random tensors for ``cfg``, scaled so that activations stay of order one."""
    g = torch.Generator().manual_seed(seed)
    width, W = cfg["width"], {}

    def rnd(*shape, scale=1.0):
        return (torch.randn(*shape, generator=g, dtype=torch.float64) * scale).to(dtype)

    def lin(out, inp, gain=1.0):
        return rnd(out, inp, scale=gain / math.sqrt(inp))

    W["embed"], W["head"] = rnd(cfg["vocab"], width), lin(cfg["vocab"], width)
    W["final.norm"], W["final.norm.b"] = 1 + rnd(width, scale=0.1), rnd(width, scale=0.1)
    S = cfg.get("streams")
    for i, L in enumerate(cfg["layers"]):
        p = f"l{i}."
        for q in (1, 2):
            if q == 2 and not L.get("mlp"):
                continue
            W[f"{p}norm{q}"], W[f"{p}norm{q}.b"] = 1 + rnd(width, scale=0.1), rnd(width, scale=0.1)
            W[f"{p}ls{q}"] = 0.5 + rnd(width, scale=0.1)
            if S is not None:
                W[f"{p}hc{q}.in"] = 1.0 / S + rnd(S, scale=0.1)
                W[f"{p}hc{q}.out"] = 1 + rnd(S, scale=0.2)
                W[f"{p}hc{q}.mix"] = torch.eye(S, dtype=dtype) + rnd(S, S, scale=0.1)
        a, r = L["mixer"]["left"], L["mixer"]["right"]
        H, G, d = a["heads"], a.get("kv_heads", a["heads"]), a["dim"]
        m = p + "mix.left."
        W[m + "q"], W[m + "q.b"], W[m + "k"], W[m + "k.b"] = lin(H * d, width), rnd(H * d, scale=0.1), lin(G * d, width), rnd(G * d, scale=0.1)
        W[m + "q.norm"], W[m + "k.norm"] = 1 + rnd(d, scale=0.2), 1 + rnd(d, scale=0.2)
        W[m + "g"], W[m + "o"], W[m + "o.b"] = lin(H, width), lin(width, H * d), rnd(width, scale=0.1)
        inner, N, R, taps = r["inner"], r["state"], r["dt_rank"], r["conv"]
        m = p + "mix.right."
        W[m + "in"], W[m + "conv"], W[m + "conv.b"] = lin(2 * inner, width), rnd(inner, taps, scale=taps ** -0.5), rnd(inner, scale=0.1)
        W[m + "x"], W[m + "dt"], W[m + "dt.b"] = lin(R + 2 * N, inner), lin(inner, R), rnd(inner, scale=0.5) - 1.0
        W[m + "A_log"] = torch.log(torch.rand(inner, N, generator=g, dtype=torch.float64) * 2 + 0.05).to(dtype)
        W[m + "D"], W[m + "o"] = rnd(inner), lin(width, inner)
        c = L.get("mlp")
        if c:
            m = p + "mlp."
            W[m + "router"] = lin(c["router"]["experts"], width, gain=2.0)
            for e in range(c["router"]["experts"]):
                ff = c["expert"]["ff"]
                W[f"{m}e{e}.gate"], W[f"{m}e{e}.up"], W[f"{m}e{e}.down"] = lin(ff, width, 2.0), lin(ff, width, 2.0), lin(width, ff)
            if c.get("shared"):
                ff = c["shared"]["ff"]
                W[m + "shared.gate"], W[m + "shared.up"], W[m + "shared.down"] = lin(ff, width, 2.0), lin(ff, width, 2.0), lin(width, ff)
                W[m + "shared.sg"] = lin(1, width)
    return W
