"""Small Porovik configurations for the tests, and helpers to write them as model folders.

A, B, C and D differ from one another in every size, constant and in the order of their layers, and avoid
coincidences: key and value sizes differ, head counts are odd or leave three query heads a key/value head,
one model has as many key/value heads as heads and no query temperature, one has forty heads on one
key/value head, value sizes and inner sizes are no multiples of 8, experts are chosen two and three at a
time, layers without a feed-forward, models that begin with a recurrent layer, value mixing between two
and three layers or none.
"""
from __future__ import annotations

import json
import os

import torch

from rosellm_b200.config.porovik import PorovikConfig
from rosellm_b200.weights import write_model_folder


def attn(heads, kv_heads, dim, vdim, scale, temp=None, v_mix=False):
    out = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "v_mix": v_mix}
    if temp is not None:
        out["q_temp"] = {"coef": temp[0], "every": temp[1]}
    return {"type": "attention", "mixer": out}


def delta(heads, dim, rank):
    return {"type": "general_delta", "mixer": {"heads": heads, "dim": dim, "decay_rank": rank}}


def gated(heads, dim, vdim):
    return {"type": "hgrn2", "mixer": {"heads": heads, "dim": dim, "vdim": vdim}}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(ff, experts, top):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}


def model(vocab, width, positions, eps, bigram, layers):
    return {"architecture": "Porovik", "vocab": vocab, "width": width, "max_positions": positions, "norm": {"eps": eps},
            "embedding": {"bigram": dict(zip(("buckets", "mul_prev", "mul_cur"), bigram))},
            "layers": [dict(l, mlp=m) for l, m in layers]}


RAW_A = model(131, 64, 512, 1e-5, (97, 31, 5), [
    (attn(6, 2, 20, 10, 0.22, temp=(0.7, 16), v_mix=True), dense(100)),
    (delta(3, 24, 5), moe(12, 5, 2)),
    (gated(2, 40, 24), None),
    (attn(4, 2, 12, 10, 0.3, temp=(0.25, 7), v_mix=True), moe(20, 6, 3)),
    (delta(2, 8, 3), dense(36)),
])
RAW_B = model(300, 96, 640, 1e-6, (211, 7, 13), [
    (gated(3, 128, 16), dense(72)),
    (attn(4, 4, 64, 32, 0.125), moe(40, 4, 1)),
    (delta(2, 64, 16), None),
    (attn(2, 2, 24, 72, 0.2, temp=(1.5, 64)), dense(64)),
])
RAW_C = model(77, 48, 700, 1e-4, (50, 3, 1), [
    (delta(1, 16, 40), moe(8, 3, 2)),
    (attn(40, 1, 8, 8, 0.35, temp=(0.1, 1), v_mix=True), dense(20)),
    (attn(5, 1, 16, 8, 0.25, v_mix=True), None),
    (gated(4, 12, 20), moe(16, 8, 3)),
    (attn(2, 1, 40, 8, 0.15, temp=(0.4, 100), v_mix=True), dense(24)),
])
RAW_D = model(2000, 384, 1024, 1e-5, (1499, 1031, 17), [
    (attn(12, 4, 48, 80, 0.14, temp=(0.5, 32), v_mix=True), moe(96, 8, 2)),
    (gated(6, 64, 96), dense(640)),
    (delta(6, 64, 24), moe(128, 4, 1)),
    (attn(12, 4, 48, 80, 0.14, temp=(0.5, 32), v_mix=True), dense(512)),
    (delta(3, 96, 8), None),
    (gated(2, 32, 136), moe(64, 16, 4)),
])
# No attention at all (no cache of keys: state slots only), and attention only, with seven heads on seven
# key/value heads of odd sizes.
RAW_E = model(90, 40, 600, 1e-5, (64, 5, 9), [
    (gated(5, 8, 8), moe(8, 4, 2)),
    (delta(2, 20, 6), dense(16)),
])
RAW_F = model(64, 56, 600, 1e-5, (61, 1, 0), [
    (attn(7, 7, 9, 5, 0.33, temp=(2.0, 3)), None),
    (attn(8, 1, 6, 12, 0.4, v_mix=True), dense(40)),
    (attn(4, 2, 10, 6, 0.3, v_mix=True), None),   # as many value entries a token, cut into other heads
])
TINY = {
    "A": dict(raw=RAW_A, seed=21, std=0.2, page_size=16),
    "B": dict(raw=RAW_B, seed=22, std=0.15, page_size=8),
    "C": dict(raw=RAW_C, seed=23, std=0.25, page_size=32),
    "D": dict(raw=RAW_D, seed=24, std=0.07, page_size=16),
    "E": dict(raw=RAW_E, seed=25, std=0.3, page_size=16),
    "F": dict(raw=RAW_F, seed=26, std=0.2, page_size=8),
}
# A wide one, for the products' tensor-core paths, contexts of many key tiles and states of 64 and 128
# columns: sixteen heads on four key/value heads of 64/64, a delta rule of 16 x 64 x 64, a gated
# recurrence of 8 x 128 x 128, sixteen experts of 512.  Not among the models every test runs on.
RAW_WIDE = model(3000, 1024, 1024, 1e-5, (65521, 36313, 27191), [
    (attn(16, 4, 64, 64, 0.125, temp=(0.5, 128), v_mix=True), dense(2048)),
    (delta(16, 64, 64), moe(512, 16, 2)),
    (gated(8, 128, 128), dense(2048)),
    (attn(16, 4, 64, 64, 0.125, temp=(0.5, 128), v_mix=True), moe(512, 16, 2)),
])
WIDE = dict(raw=RAW_WIDE, seed=31, std=0.03, page_size=16)


def write_tiny(name: str, root: str, decisive: bool = False) -> str:
    """A model folder of random weights.  The lower bounds of the forget gates are spread over (0, 0.9),
    the value-mixing weights over (0.2, 0.8), the decays' and gates' biases over a few units.
    ``decisive`` (the folders of the 16-bit runs): a layer's experts are made near copies of its first
    (nine parts of it, one part their own), so that a choice of experts which is a close call, and
    which 16-bit rounding turns, changes the logits no more than rounding does; with experts that have
    nothing in common every such token, and in a model with recurrent layers every token after it,
    would differ by more than any rounding bound, which says nothing about the engine.  Choices among
    unlike experts are what the 32-bit runs test."""
    from safetensors.torch import load_file, save_file

    t = WIDE if name == "WIDE" else TINY[name]
    out = os.path.join(root, f"porovik_{name}" + ("_decisive" if decisive else ""))
    if not os.path.isfile(os.path.join(out, "model.safetensors")):
        write_model_folder(PorovikConfig.from_dict(t["raw"]), t["seed"], out, std=t["std"], norm_affine="random")
        path = os.path.join(out, "model.safetensors")
        tensors = load_file(path)
        g = torch.Generator().manual_seed(t["seed"])
        for key in sorted(tensors):
            old = tensors[key]
            if key.endswith("mix.lower"):
                tensors[key] = (torch.rand(old.shape, generator=g) * 0.9).to(old.dtype)
            elif key.endswith("mix.vmix"):
                tensors[key] = (0.2 + 0.6 * torch.rand(old.shape, generator=g)).to(old.dtype)
            elif key.endswith(("mix.w0", "mix.a.b", "mix.f.b")):
                tensors[key] = (torch.randn(old.shape, generator=g) * 1.5).to(old.dtype)
            elif decisive and ".mlp.e" in key and ".mlp.e0." not in key:
                first = tensors[key[:key.index(".mlp.e")] + ".mlp.e0." + key.rsplit(".", 1)[1]]
                tensors[key] = (0.9 * first.float() + 0.1 * old.float()).to(old.dtype)
        save_file(tensors, path)
    return out


def load_folder(folder: str):
    from safetensors.torch import load_file

    with open(os.path.join(folder, "config.json")) as f:
        cfg = json.load(f)
    return cfg, load_file(os.path.join(folder, "model.safetensors"))
