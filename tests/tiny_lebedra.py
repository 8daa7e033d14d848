"""Small Lebedra configurations for the tests, and helpers to write them as model folders.

X, Y, Z and W differ from one another in every size and option, and avoid coincidences: the plain
and rotated query parts have different sizes, value and latent sizes differ from both, head
counts are odd, a group keeps more than one of several groups, inner sizes and the token
input's size are no multiples of 8, and one layer has no feed-forward.
"""
from __future__ import annotations

import json
import os

from rosellm_b200.config.lebedra import LebedraConfig
from rosellm_b200.weights import write_model_folder


def mixer(heads, dim, rot_dim, vdim, kv_rank, scale, base, dims=None):
    return {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "scale": scale,
            "rot": {"dims": rot_dim if dims is None else dims, "base": base}}


def moe(ff, limit, experts, top, count=None, keep=None):
    router = {"experts": experts, "top": top}
    if count is not None:
        router["groups"] = {"count": count, "keep": keep}
    return {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": router}


RAW_X = {
    "architecture": "Lebedra", "vocab": 300, "width": 64, "residual_mult": 0.7, "norm": {"eps": 1e-5},
    "token_side": {"dim": 12},
    "layers": [
        {"type": "latent_attention", "mixer": mixer(3, 16, 8, 24, 40, 0.3, 100.0), "mlp": {"kind": "dense", "ff": 100}},
        {"type": "latent_attention", "mixer": mixer(5, 8, 16, 12, 20, 0.45, 10000.0), "mlp": moe(24, 0.8, 12, 3, 4, 2)},
        {"type": "latent_attention", "mixer": mixer(2, 24, 4, 16, 56, 0.2, 500.0, dims=2), "mlp": None},
        {"type": "latent_attention", "mixer": mixer(3, 16, 8, 24, 40, 0.3, 100.0), "mlp": moe(20, 2.5, 6, 2, 3, 1)},
    ],
}
RAW_Y = {
    "architecture": "Lebedra", "vocab": 777, "width": 96, "residual_mult": 1.0, "norm": {"eps": 1e-6},
    "token_side": None,
    "layers": [
        {"type": "latent_attention", "mixer": mixer(1, 32, 32, 48, 24, 0.125, 1e6), "mlp": moe(40, 1.5, 4, 1)},
        {"type": "latent_attention", "mixer": mixer(7, 8, 2, 8, 16, 0.5, 50.0), "mlp": {"kind": "dense", "ff": 72}},
    ],
}
# Sizes that are multiples of nothing convenient: per-head sizes of 12, 6 and 10, a latent of 18,
# five experts, an inner size of 36 and 12, a token input of 5 entries, a prime vocabulary.
RAW_Z = {
    "architecture": "Lebedra", "vocab": 131, "width": 72, "residual_mult": 0.3, "norm": {"eps": 1e-4},
    "token_side": {"dim": 5},
    "layers": [
        {"type": "latent_attention", "mixer": mixer(3, 12, 6, 10, 18, 0.4, 20.0), "mlp": moe(12, 1.0, 5, 2)},
        {"type": "latent_attention", "mixer": mixer(9, 4, 10, 6, 30, 0.35, 7.0), "mlp": {"kind": "dense", "ff": 36}},
    ],
}
# A wider one: six and twelve heads, latents of 96 and 128, eight experts, a layer without a
# feed-forward in the middle.
RAW_W = {
    "architecture": "Lebedra", "vocab": 2000, "width": 384, "residual_mult": 0.4, "norm": {"eps": 1e-5},
    "token_side": {"dim": 40},
    "layers": [
        {"type": "latent_attention", "mixer": mixer(6, 48, 16, 56, 96, 0.11, 1e4), "mlp": {"kind": "dense", "ff": 640}},
        {"type": "latent_attention", "mixer": mixer(6, 48, 16, 56, 96, 0.11, 1e4), "mlp": moe(256, 2.0, 8, 2, 4, 2)},
        {"type": "latent_attention", "mixer": mixer(12, 32, 32, 32, 128, 0.1, 5e5), "mlp": None},
        {"type": "latent_attention", "mixer": mixer(6, 48, 16, 56, 96, 0.11, 1e4), "mlp": moe(192, 1.0, 8, 3, 2, 2)},
    ],
}
TINY = {
    "X": dict(raw=RAW_X, seed=11, std=0.2, page_size=16),
    "Y": dict(raw=RAW_Y, seed=12, std=0.25, page_size=8),
    "Z": dict(raw=RAW_Z, seed=13, std=0.2, page_size=32),
    "W": dict(raw=RAW_W, seed=14, std=0.08, page_size=16),
}


def write_tiny(name: str, root: str, decisive: bool = False) -> str:
    """``decisive``: the routers' choice corrections are set further apart (steps of 2, half of
    them negative) than two scores can be, so that no token's choice of experts or groups is a
    close call that 16-bit rounding could turn; the chosen experts' weights still depend on the
    token.  (Choices that depend on the token are what the 32-bit runs of the other folders test.)"""
    t = TINY[name]
    out = os.path.join(root, f"lebedra_{name}" + ("_decisive" if decisive else ""))
    if not os.path.isfile(os.path.join(out, "model.safetensors")):
        write_model_folder(LebedraConfig.from_dict(t["raw"]), t["seed"], out, std=t["std"], norm_affine="random")
        if decisive:
            import torch
            from safetensors.torch import load_file, save_file

            path = os.path.join(out, "model.safetensors")
            tensors = load_file(path)
            g = torch.Generator().manual_seed(t["seed"])
            for key in sorted(tensors):
                if key.endswith("mlp.correction"):
                    n = tensors[key].numel()
                    tensors[key] = (torch.randperm(n, generator=g).float() * 2.0 - n).to(tensors[key].dtype)
            save_file(tensors, path)
    return out


def load_folder(folder: str):
    from safetensors.torch import load_file

    with open(os.path.join(folder, "config.json")) as f:
        cfg = json.load(f)
    return cfg, load_file(os.path.join(folder, "model.safetensors"))
