"""Porovik, plain and slow: whole sequences, no cache, no batch, float64, one function per mechanism.

Written from the design's equations only; it shares no code with the package.  Notation: ``h`` the
normalised input of a sublayer [tokens, width], ``W[name]`` a tensor of the weight file, positions count
from 0.
"""
from __future__ import annotations

import math

import torch

F64 = torch.float64


def rms(x, eps):
    return x / torch.sqrt(x.pow(2).mean(-1, keepdim=True) + eps)


def norm(x, w, eps):
    """The file holds a scale as its offset from one."""
    return rms(x, eps) * (1.0 + w)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z):
    return z * torch.sigmoid(z)


def embed(tokens, table, pair_table, pos_table, buckets, mul_prev, mul_cur):
    rows = [buckets if p == 0 else (tokens[p - 1] * mul_prev + t * mul_cur) % buckets for p, t in enumerate(tokens)]
    return table[tokens] + pair_table[rows] + pos_table[: len(tokens)]


def attention(q, k, v, scale, slopes, temp):
    """q [n, H, dk], k [n, G, dk], v [n, G, dv]; temp [n] multiplies the queries; slopes [H]."""
    n, H, _ = q.shape
    G = k.shape[1]
    i = torch.arange(n)[:, None]
    j = torch.arange(n)[None, :]
    out = torch.zeros(n, H, v.shape[2], dtype=F64)
    for h in range(H):
        g = h // (H // G)
        s = ((q[:, h] * temp[:, None]) @ k[:, g].T) * scale - slopes[h] * (i - j).to(F64)
        s = s.masked_fill(j > i, -math.inf)
        out[:, h] = torch.softmax(s, dim=-1) @ v[:, g]
    return out


def query_temperature(n, coef, every):
    if not every:
        return torch.ones(n, dtype=F64)
    p = torch.arange(n)
    return 1.0 + coef * torch.log(((p + 1) // every + 1).to(F64))


def distance_slopes(H):
    return torch.tensor([2.0 ** (-8.0 * (h + 1) / H) for h in range(H)], dtype=F64)


def attention_mixer(h, W, p, mx, v_first):
    """Returns (mixer output, the values as they are cached, v_first for later layers)."""
    n = h.shape[0]
    H, G, dk, dv = mx["heads"], mx.get("kv_heads", mx["heads"]), mx["dim"], mx["vdim"]
    q = (h @ W[p + "q"].T).view(n, H, dk)
    k = (h @ W[p + "k"].T).view(n, G, dk)
    v = (h @ W[p + "v"].T).view(n, G, dv)
    if mx.get("v_mix"):
        if v_first is None:
            v_first = v
        else:
            lam = W[p + "vmix"]
            v = (1.0 - lam) * v + lam * v_first.reshape(v.shape)  # entry by entry of a token's values
    qt = mx.get("q_temp") or {}
    o = attention(q, k, v, mx["scale"], distance_slopes(H), query_temperature(n, qt.get("coef", 0.0), qt.get("every", 0)))
    o = o.reshape(n, H * dv) * torch.sigmoid(h @ W[p + "g"].T)
    return o @ W[p + "o"].T, v_first


def delta_rule(r, k, v, w, a, unit_eps=1e-6):
    """One head.  r, k, v, w, a: [n, d].  Returns o [n, d]."""
    n, d = r.shape
    S = torch.zeros(d, d, dtype=F64)
    out = torch.zeros(n, d, dtype=F64)
    for t in range(n):
        u = k[t] / torch.sqrt(k[t].pow(2).sum() + unit_eps)
        old = S
        S = w[t][:, None] * old - torch.outer(a[t] * u, u @ old) + torch.outer(k[t], v[t])
        out[t] = S.T @ r[t]
    return out


def delta_mixer(h, W, p, mx, eps):
    n = h.shape[0]
    H, d = mx["heads"], mx["dim"]
    r, k, v = (h @ W[p + "r"].T).view(n, H, d), (h @ W[p + "k"].T).view(n, H, d), (h @ W[p + "v"].T).view(n, H, d)
    w = torch.exp(-math.exp(-0.5) * torch.sigmoid(torch.tanh(h @ W[p + "w1"].T) @ W[p + "w2"].T + W[p + "w0"])).view(n, H, d)
    a = torch.sigmoid(h @ W[p + "a"].T + W[p + "a.b"]).view(n, H, d)
    o = torch.stack([delta_rule(r[:, i], k[:, i], v[:, i], w[:, i], a[:, i]) for i in range(H)], dim=1)
    o = rms(o, eps).reshape(n, H * d) * W[p + "norm"] * torch.sigmoid(h @ W[p + "g"].T)
    return o @ W[p + "o"].T


def gated_recurrence(q, f, v):
    """One head.  q, f: [n, dk]; v: [n, dv]."""
    n, dk = q.shape
    S = torch.zeros(dk, v.shape[1], dtype=F64)
    out = torch.zeros(n, v.shape[1], dtype=F64)
    for t in range(n):
        S = f[t][:, None] * S + torch.outer(1.0 - f[t], v[t])
        out[t] = S.T @ q[t]
    return out


def gated_mixer(h, W, p, mx, eps):
    n = h.shape[0]
    H, dk, dv = mx["heads"], mx["dim"], mx["vdim"]
    q = silu(h @ W[p + "q"].T).view(n, H, dk)
    v = (h @ W[p + "v"].T).view(n, H, dv)
    low = W[p + "lower"]
    f = (low + (1.0 - low) * torch.sigmoid(h @ W[p + "f"].T + W[p + "f.b"])).view(n, H, dk)
    o = torch.stack([gated_recurrence(q[:, i], f[:, i], v[:, i]) for i in range(H)], dim=1)
    o = rms(o, eps) * W[p + "norm"]
    return o.reshape(n, H * dv) @ W[p + "o"].T


def dense_ff(h, W, p):
    return (gelu_tanh(h @ W[p + "gate"].T) * (h @ W[p + "up"].T)) @ W[p + "down"].T


def route(h, router, top):
    """(chosen experts [n, top], their scores): sigmoid scores, the largest first, ties to the lower index."""
    s = torch.sigmoid(h @ router.T)
    order = torch.sort(s, dim=-1, descending=True, stable=True).indices[:, :top]
    return order, torch.gather(s, 1, order)


def moe_ff(h, W, p, ml):
    idx, val = route(h, W[p + "router"], ml["router"]["top"])
    y = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, s in zip(idx[t].tolist(), val[t]):
            x = s * h[t]
            q = f"{p}e{e}."
            y[t] += (silu(W[q + "gate"] @ x) * (W[q + "up"] @ x)) @ W[q + "down"].T
    return y


def forward(cfg, weights, tokens, layers_out=None):
    """Logits [tokens, vocab] of one sequence."""
    W = {k: v.to(F64) for k, v in weights.items()}
    eps = cfg["norm"]["eps"]
    bg = cfg["embedding"]["bigram"]
    x = embed(list(tokens), W["embed"], W["bigram"], W["pos"], bg["buckets"], bg["mul_prev"], bg["mul_cur"])
    v_first = None
    for i, lc in enumerate(cfg["layers"]):
        p = f"l{i}."
        h = norm(x, W[p + "norm1"], eps)
        if lc["type"] == "attention":
            y, v_first = attention_mixer(h, W, p + "mix.", lc["mixer"], v_first)
        elif lc["type"] == "general_delta":
            y = delta_mixer(h, W, p + "mix.", lc["mixer"], eps)
        else:
            y = gated_mixer(h, W, p + "mix.", lc["mixer"], eps)
        x = x + norm(y, W[p + "norm1b"], eps)
        ml = lc.get("mlp")
        if ml is not None:
            h = norm(x, W[p + "norm2"], eps)
            y = dense_ff(h, W, p + "mlp.") if ml["kind"] == "dense" else moe_ff(h, W, p + "mlp.", ml)
            x = x + norm(y, W[p + "norm2b"], eps)
        if layers_out is not None:
            layers_out.append(x.clone())
    return norm(x, W["final.norm"], eps) @ W["embed"].T
