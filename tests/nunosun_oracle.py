"""A plain, slow evaluation of the Nunosun design in float64, one function per mechanism, for the tests.

Nothing here is shared with the product path: no framework import, whole sequences only, no cache, no state carried between
calls.  ``W`` maps checkpoint tensor names to tensors (``l<i>.mix.*``, ``l<i>.mlp.*`` ...); linear weights are ``[out, in]``.

Notation: ``x`` is the residual stream ``[T, width]``; ``n(x) = x / sqrt(mean(x^2) + eps)``.

    x0 = n(E[tok]) * w_e
    per layer:  h = n(x) * w1;   m = h + conv(h);   x <- x + mixer(m) + ff(h);   x <- x + n(P (gelu(G x) * e_tok)) * w_s
    logits = (n(x) * w_f) H^T * logit_scale
"""
import math

import torch

F64 = torch.float64


def rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def silu(z):
    return z / (1.0 + torch.exp(-z))


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def softplus(z):
    return torch.where(z > 30, z, torch.log1p(torch.exp(torch.clamp(z, max=30))))


def causal_conv(x, w):
    """``y_t = sum_j w[:, j] x_(t - taps + 1 + j)`` per channel, zeros before the start.  ``x [T, C]``, ``w [C, taps]``."""
    T, taps = x.shape[0], w.shape[1]
    y = torch.zeros_like(x)
    for t in range(T):
        for j in range(taps):
            s = t - taps + 1 + j
            if s >= 0:
                y[t] += w[:, j] * x[s]
    return y


def bucket(n, B, D):
    """The row of the bias table for distance ``n``: one row each below ``B // 2``, then logarithmic steps up to ``D``."""
    half = B // 2
    if n < half:
        return n
    return min(B - 1, half + int(math.floor(math.log(n / half) / math.log(D / half) * (B - half))))


def window_attention(q, k, v, scale, window, rel=None, bias_max=0.0, first=0):
    """``q [n, H, d]`` are the queries of positions ``first .. first + n - 1``; ``k [L, G, d]``, ``v [L, G, dv]`` hold all
    positions from 0.  Position ``i`` sees ``j`` with ``0 <= i - j < window`` (``window = 0``: every ``j <= i``); the score is
    ``q . k * scale + rel[bucket(i - j), h]``; plain softmax.  Returns ``[n, H, dv]``."""
    n, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros(n, H, v.shape[2], dtype=F64)
    for a in range(n):
        i = first + a
        lo = max(0, i - window + 1) if window > 0 else 0
        for h in range(H):
            g = h // (H // G)
            s = (k[lo:i + 1, g] @ q[a, h]) * scale
            if rel is not None:
                s = s + torch.stack([rel[bucket(i - j, rel.shape[0], bias_max), h] for j in range(lo, i + 1)])
            p = torch.exp(s - s.max())
            out[a, h] = (p / p.sum()) @ v[lo:i + 1, g]
    return out


def rotate_half(x, positions, dims, base):
    """Turn the first ``dims`` entries of every head of ``x [T, H, d]``: entry ``i`` with entry ``i + dims / 2`` by the angle
    ``position * base^(-2 i / dims)``."""
    if not dims:
        return x
    y = x.clone()
    half = dims // 2
    for t, pos in enumerate(positions):
        for i in range(half):
            ang = pos * base ** (-2.0 * i / dims)
            c, s = math.cos(ang), math.sin(ang)
            u, w = x[t, :, i], x[t, :, i + half]
            y[t, :, i] = u * c - w * s
            y[t, :, i + half] = w * c + u * s
    return y


def retention(q, k, v, decay):
    """``S <- decay_h S + k v^T``, ``o = S^T q`` from a zero memory; ``q, k [T, H, d]``, ``v [T, H, dv]``."""
    T, H, d = q.shape
    S = torch.zeros(H, d, v.shape[2], dtype=F64)
    out = torch.zeros(T, H, v.shape[2], dtype=F64)
    for t in range(T):
        for h in range(H):
            S[h] = decay[h] * S[h] + torch.outer(k[t, h], v[t, h])
            out[t, h] = S[h].T @ q[t, h]
    return out


def delta_rule(q, k, v, g, beta):
    """Per head: ``S <- g S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q``.  ``q, k [T, H, d]`` (already expanded to
    the value heads), ``v [T, H, dv]``, ``g, beta [T, H]``."""
    T, H, d = q.shape
    S = torch.zeros(H, d, v.shape[2], dtype=F64)
    out = torch.zeros(T, H, v.shape[2], dtype=F64)
    for t in range(T):
        for h in range(H):
            S[h] = g[t, h] * S[h]
            u = beta[t, h] * (v[t, h] - S[h].T @ k[t, h])
            S[h] = S[h] + torch.outer(k[t, h], u)
            out[t, h] = S[h].T @ q[t, h]
    return out


def unit(x, eps=1e-6):
    return x / torch.sqrt((x * x).sum(-1, keepdim=True) + eps)


def poly_norm(z, coef, eps):
    return coef[0] * rms(z, eps) + coef[1] * rms(z * z, eps) + coef[2] * rms(z * z * z, eps) + coef[3]


def route(z, top):
    """``z [E]`` -> (chosen experts, their weights): the ``top`` largest logits, softmax over those alone."""
    idx = sorted(range(z.shape[0]), key=lambda e: -float(z[e]))[:top]
    w = torch.exp(z[idx] - z[idx].max())
    return idx, w / w.sum()


# -- mixers and feed-forwards from the checkpoint's tensors -------------------------------------------------------------
def attention_mixer(m, W, p, c, eps):
    T = m.shape[0]
    H, G, d, dv = c["heads"], c.get("kv_heads", c["heads"]), c["dim"], c.get("vdim", c["dim"])
    q = rms((m @ W[p + "q"].T).view(T, H, d), eps) * W[p + "q.norm"]
    k = rms((m @ W[p + "k"].T).view(T, G, d), eps) * W[p + "k.norm"]
    v = (m @ W[p + "v"].T).view(T, G, dv)
    o = window_attention(q, k, v, c["scale"], (c.get("mask") or {}).get("size", 0), W.get(p + "rel"), c.get("bias_max", 0.0))
    return o.reshape(T, H * dv) @ W[p + "o"].T


def retention_mixer(m, W, p, c, eps):
    T = m.shape[0]
    H, d, dv = c["heads"], c["dim"], c.get("vdim", c["dim"])
    rot = c.get("rot") or {}
    pos = list(range(T))
    q = rotate_half((m @ W[p + "q"].T).view(T, H, d), pos, rot.get("dims", 0), rot.get("base", 10000.0))
    k = rotate_half((m @ W[p + "k"].T).view(T, H, d), pos, rot.get("dims", 0), rot.get("base", 10000.0)) * d ** -0.5
    v = (m @ W[p + "v"].T).view(T, H, dv)
    o = rms(retention(q, k, v, c["decay"]), eps).reshape(T, H * dv) * silu(m @ W[p + "g"].T)
    return o @ W[p + "o"].T


def delta_mixer(m, W, p, c, eps):
    T = m.shape[0]
    H, G, d, dv = c["heads"], c.get("kv_heads", c["heads"]), c["dim"], c.get("vdim", c["dim"])
    q = silu(causal_conv(m @ W[p + "q"].T, W[p + "q.conv"])).view(T, G, d)
    k = silu(causal_conv(m @ W[p + "k"].T, W[p + "k.conv"])).view(T, G, d)
    v = silu(causal_conv(m @ W[p + "v"].T, W[p + "v.conv"])).view(T, H, dv)
    q, k = unit(q) * d ** -0.5, unit(k)
    rep = H // G
    q, k = q.repeat_interleave(rep, dim=1), k.repeat_interleave(rep, dim=1)
    beta = 1.0 / (1.0 + torch.exp(-(m @ W[p + "b"].T)))
    g = torch.exp(-torch.exp(W[p + "A_log"]) * softplus(m @ W[p + "a"].T + W[p + "dt_bias"]))
    o = rms(delta_rule(q, k, v, g, beta), eps) * W[p + "norm"]
    return (o.reshape(T, H * dv) * silu(m @ W[p + "g"].T)) @ W[p + "o"].T


def feed_forward(h, W, p, c, eps):
    if not c:
        return torch.zeros_like(h)
    if c.get("kind", "dense") == "dense":
        return poly_norm(h @ W[p + "up"].T, W[p + "act"], eps) @ W[p + "down"].T
    out = torch.zeros_like(h)
    logits = h @ W[p + "router"].T + W[p + "router.b"]
    for t in range(h.shape[0]):
        idx, w = route(logits[t], c["router"]["top"])
        for e, we in zip(idx, w):
            pe = f"{p}e{e}."
            out[t] += we * ((silu(W[pe + "gate"] @ h[t]) * (W[pe + "up"] @ h[t])) @ W[pe + "down"].T)
    return out


def forward(cfg, W, tokens, return_layers=False):
    """Logits ``[T, vocab]`` of a whole sequence (and the stream after every layer)."""
    W = {k: v.to(F64) for k, v in W.items()}
    eps = cfg["norm"]["eps"]
    tok = torch.tensor(tokens)
    x = rms(W["embed"][tok], eps) * W["embed.norm"]
    sd = (cfg.get("token_side") or {}).get("dim", 0)
    taps = (cfg.get("canon") or {}).get("taps", 0)
    layers = []
    for i, l in enumerate(cfg["layers"]):
        p = f"l{i}."
        h = rms(x, eps) * W[p + "norm1"]
        m = h + causal_conv(h, W[p + "canon1"]) if taps > 1 else h
        if l["type"] == "parallel":
            a = attention_mixer(m, W, p + "mix.left.", l["mixer"]["left"], eps)
            b = retention_mixer(m, W, p + "mix.right.", l["mixer"]["right"], eps)
            mix = 0.5 * (rms(a, eps) * W[p + "mix.left.out"] + rms(b, eps) * W[p + "mix.right.out"])
        else:
            mix = delta_mixer(m, W, p + "mix.", l["mixer"], eps)
        x = x + (mix + feed_forward(h, W, p + "mlp.", l.get("mlp"), eps))
        if sd:
            e = W["side.embed"][tok][:, i * sd:(i + 1) * sd]
            y = (gelu_tanh(x @ W[p + "side.gate"].T) * e) @ W[p + "side.proj"].T
            x = x + rms(y, eps) * W[p + "side.norm"]
        layers.append(x.clone())
    logits = (rms(x, eps) * W["final.norm"]) @ W["head"].T * cfg.get("logit_scale", 1.0)
    return (logits, layers) if return_layers else logits


# -- random checkpoints ---------------------------------------------------------------------------------------------------
def random_weights(cfg, seed=0, bias_buckets=10):
    """Every tensor a checkpoint of ``cfg`` holds, fp32, from ``seed``: projections scaled by ``fan_in^-1/2``, norm weights
    around one, gates and biases spread enough that every branch matters."""
    g = torch.Generator().manual_seed(seed)
    Wd, V = cfg["width"], cfg["vocab"]
    n_layers = len(cfg["layers"])
    sd = (cfg.get("token_side") or {}).get("dim", 0)
    taps = (cfg.get("canon") or {}).get("taps", 0)

    def lin(o, i, s=1.0):
        return torch.randn(o, i, generator=g) * (s * i ** -0.5)

    def around_one(n):
        return 1.0 + 0.2 * torch.randn(n, generator=g)

    W = {"embed": torch.randn(V, Wd, generator=g), "embed.norm": around_one(Wd), "final.norm": around_one(Wd), "head": lin(V, Wd)}
    if sd:
        W["side.embed"] = torch.randn(V, n_layers * sd, generator=g)
    for i, l in enumerate(cfg["layers"]):
        p = f"l{i}."
        W[p + "norm1"] = around_one(Wd)
        if taps > 1:
            W[p + "canon1"] = torch.randn(Wd, taps, generator=g) * 0.4
        if sd:
            W[p + "side.gate"], W[p + "side.proj"], W[p + "side.norm"] = lin(sd, Wd), lin(Wd, sd), around_one(Wd) * 0.5
        mx = l["mixer"]
        if l["type"] == "delta":
            H, G, d, dv, ct = mx["heads"], mx.get("kv_heads", mx["heads"]), mx["dim"], mx.get("vdim", mx["dim"]), mx.get("conv", 1)
            q = p + "mix."
            for n_, rows in (("q", G * d), ("k", G * d), ("v", H * dv)):
                W[q + n_] = lin(rows, Wd, 2.0)
                W[q + n_ + ".conv"] = torch.randn(rows, ct, generator=g) * 0.6
            W[q + "b"], W[q + "a"], W[q + "g"], W[q + "o"] = lin(H, Wd, 2.0), lin(H, Wd, 2.0), lin(H * dv, Wd, 2.0), lin(Wd, H * dv)
            W[q + "A_log"] = torch.randn(H, generator=g) * 0.5 - 1.0
            W[q + "dt_bias"] = torch.randn(H, generator=g) * 0.5
            W[q + "norm"] = around_one(dv)
        else:
            a, r = mx["left"], mx["right"]
            H, G, d, dv = a["heads"], a.get("kv_heads", a["heads"]), a["dim"], a.get("vdim", a["dim"])
            q = p + "mix.left."
            W[q + "q"], W[q + "k"], W[q + "v"], W[q + "o"] = lin(H * d, Wd, 2.0), lin(G * d, Wd, 2.0), lin(G * dv, Wd), lin(Wd, H * dv)
            W[q + "q.norm"], W[q + "k.norm"] = around_one(d) * 1.5, around_one(d) * 1.5
            if "bias_max" in a:
                W[q + "rel"] = torch.randn(a.get("bias_buckets", bias_buckets), H, generator=g)
            W[q + "out"] = around_one(Wd)
            H, d, dv = r["heads"], r["dim"], r.get("vdim", r["dim"])
            q = p + "mix.right."
            W[q + "q"], W[q + "k"], W[q + "v"], W[q + "g"], W[q + "o"] = (lin(H * d, Wd), lin(H * d, Wd), lin(H * dv, Wd), lin(H * dv, Wd, 2.0),
                                                                         lin(Wd, H * dv))
            W[q + "out"] = around_one(Wd)
        mlp = l.get("mlp")
        if not mlp:
            continue
        q = p + "mlp."
        if mlp.get("kind", "dense") == "dense":
            W[q + "up"], W[q + "down"] = lin(mlp["ff"], Wd), lin(Wd, mlp["ff"])
            W[q + "act"] = torch.tensor([0.8, 0.4, -0.3, 0.1]) + 0.1 * torch.randn(4, generator=g)
        else:
            E, ff = mlp["router"]["experts"], mlp["expert"]["ff"]
            W[q + "router"], W[q + "router.b"] = lin(E, Wd, 3.0), torch.randn(E, generator=g)
            for e in range(E):
                W[f"{q}e{e}.gate"], W[f"{q}e{e}.up"], W[f"{q}e{e}.down"] = lin(ff, Wd, 2.0), lin(ff, Wd), lin(Wd, ff)
    return W
