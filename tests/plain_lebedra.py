"""A plain, slow Lebedra: whole sequences on the CPU, no cache, one function per mechanism.

Everything is written out from the design's equations in float64 or float32 torch
operations on whole sequences; nothing here is shared with the package's parts or kernels.
``weights`` is a dict of tensors by file name, ``cfg`` the ``config.json`` dictionary.
"""
from __future__ import annotations

import math

import torch


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def unit_rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    return unit_rms(x, eps) * w


def rotate_pairs(v: torch.Tensor, positions: torch.Tensor, dims: int, base: float) -> torch.Tensor:
    """``v`` [tokens, ..., width]: the first ``dims`` entries of the last axis are turned pair by
    pair, (2i, 2i+1) by the angle position * base^(-2i/dims); the rest stay."""
    out = v.clone()
    half = dims // 2
    i = torch.arange(half, dtype=v.dtype)
    freq = base ** (-2.0 * i / dims)
    ang = positions.to(v.dtype)[:, None] * freq[None, :]          # [tokens, half]
    shape = [v.shape[0]] + [1] * (v.dim() - 2) + [half]
    c, s = torch.cos(ang).view(shape), torch.sin(ang).view(shape)
    a, b = v[..., 0:dims:2], v[..., 1:dims:2]
    out[..., 0:dims:2] = a * c - b * s
    out[..., 1:dims:2] = b * c + a * s
    return out


def softmax_with_sink(scores: torch.Tensor, sink: torch.Tensor) -> torch.Tensor:
    """``scores`` [heads, queries, keys] with -inf where a key is hidden; ``sink`` [heads]: one
    more term exp(sink) in each row's denominator, with no value behind it."""
    top = torch.maximum(scores.max(dim=-1).values, sink[:, None].expand(scores.shape[:2]))
    e = torch.exp(scores - top[..., None])
    return e / (e.sum(dim=-1) + torch.exp(sink[:, None] - top))[..., None]


def latent_attention(h: torch.Tensor, w: dict, p: str, mix: dict, eps: float) -> torch.Tensor:
    """The mixer on a whole sequence ``h`` [tokens, width], expanded keys and values per head."""
    n = h.shape[0]
    H, d, r, dv, rank = mix["heads"], mix["dim"], mix["rot_dim"], mix["vdim"], mix["kv_rank"]
    pos = torch.arange(n)
    q = (h @ w[p + "q"].T).view(n, H, d + r)
    q_plain, q_rot = q[..., :d], q[..., d:]
    dkv = h @ w[p + "dkv"].T
    c = rms_norm(dkv[:, :rank], w[p + "dkv.norm"], eps)
    k_rot = dkv[:, rank:]
    rot = mix["rot"]
    q_rot = rotate_pairs(q_rot, pos, rot["dims"], rot["base"])
    k_rot = rotate_pairs(k_rot, pos, rot["dims"], rot["base"])
    k_plain = (c @ w[p + "uk"].T).view(n, H, d)
    v = (c @ w[p + "uv"].T).view(n, H, dv)
    scores = torch.einsum("qhd,khd->hqk", q_plain, k_plain) + torch.einsum("qhr,kr->hqk", q_rot, k_rot)
    scores = scores * mix["scale"]
    hidden = torch.arange(n)[None, :] > torch.arange(n)[:, None]
    scores = scores.masked_fill(hidden[None], float("-inf"))
    prob = softmax_with_sink(scores, w[p + "sink"].to(h.dtype))
    o = torch.einsum("hqk,khv->qhv", prob, v).reshape(n, H * dv)
    return o @ w[p + "o"].T


def dense_ff(h: torch.Tensor, w: dict, p: str) -> torch.Tensor:
    return (torch.relu(h @ w[p + "gate"].T) * (h @ w[p + "up"].T)) @ w[p + "down"].T


def expert_ff(h: torch.Tensor, w: dict, p: str, limit: float) -> torch.Tensor:
    g = torch.clamp(h @ w[p + "gate"].T, max=limit)
    u = torch.clamp(h @ w[p + "up"].T, min=-limit, max=limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ w[p + "down"].T


def route(h: torch.Tensor, w: dict, p: str, router: dict) -> tuple[torch.Tensor, torch.Tensor]:
    """Chosen experts [tokens, top] and their weights."""
    s = torch.softmax(h @ w[p + "router"].T, dim=-1)
    choice = s + w[p + "correction"].to(s.dtype)
    n_exp, top = router["experts"], router["top"]
    groups = router.get("groups")
    if groups:
        per = n_exp // groups["count"]
        best = choice.view(-1, groups["count"], per).max(dim=-1).values
        keep = best.topk(groups["keep"], dim=-1).indices
        allowed = torch.zeros_like(best, dtype=torch.bool).scatter_(1, keep, True)
        choice = choice.masked_fill(~allowed.repeat_interleave(per, dim=1), float("-inf"))
    idx = choice.topk(top, dim=-1).indices
    return idx, s.gather(1, idx)


def moe_ff(h: torch.Tensor, w: dict, p: str, mlp: dict) -> torch.Tensor:
    idx, weight = route(h, w, p, mlp["router"])
    out = torch.zeros(h.shape[0], w[p + "e0.down"].shape[0], dtype=h.dtype)
    for t in range(h.shape[0]):
        for j in range(idx.shape[1]):
            e = int(idx[t, j])
            out[t] += weight[t, j] * expert_ff(h[t:t + 1], w, f"{p}e{e}.", mlp["expert"]["limit"])[0]
    return out


def token_side(x: torch.Tensor, tokens: torch.Tensor, w: dict, layer: int, cfg: dict) -> torch.Tensor:
    """What the per-layer token input adds to the stream (before the multiplier)."""
    dim = cfg["token_side"]["dim"]
    e = w["side.embed"][tokens][:, layer * dim:(layer + 1) * dim].to(x.dtype)
    g = gelu_tanh(x @ w[f"l{layer}.side.gate"].T) * e
    return rms_norm(g @ w[f"l{layer}.side.proj"].T, w[f"l{layer}.side.norm"], cfg["norm"]["eps"])


def forward(cfg: dict, weights: dict, tokens, dtype=torch.float64, layers_out: list | None = None) -> torch.Tensor:
    """Logits [tokens, vocab] of one whole sequence; ``layers_out`` receives the stream after
    every layer."""
    w = {k: (v.to(dtype) if v.dtype.is_floating_point else v) for k, v in weights.items()}
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    eps, m = cfg["norm"]["eps"], cfg["residual_mult"]
    x = w["embed"][tokens]
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        if layer["type"] != "latent_attention":
            raise ValueError(layer["type"])
        x = x + m * rms_norm(latent_attention(x, w, p + "mix.", layer["mixer"], eps), w[p + "norm1"], eps)
        mlp = layer.get("mlp")
        if mlp is not None:
            y = dense_ff(x, w, p + "mlp.") if mlp["kind"] == "dense" else moe_ff(x, w, p + "mlp.", mlp)
            x = x + m * rms_norm(y, w[p + "norm2"], eps)
        if cfg.get("token_side"):
            x = x + m * token_side(x, tokens, w, i, cfg)
        if layers_out is not None:
            layers_out.append(x.clone())
    return rms_norm(x, w["final.norm"], eps) @ w["head"].T
