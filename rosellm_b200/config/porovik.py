"""Porovik's typed configuration, read from the keys of its own ``config.json``.

Top level: ``vocab``, ``width``, ``max_positions`` (rows of the learned position table), ``norm.eps``,
``embedding.bigram`` (``buckets``, ``mul_prev``, ``mul_cur``: the hashed table of token pairs) and
``layers``, a list whose entries give ``type`` (the mixer: ``attention``, ``general_delta`` or ``hgrn2``),
the mixer's sizes and constants under ``mixer`` and the feed-forward under ``mlp`` (null for none,
``{"kind": "dense", "ff": n}`` or ``{"kind": "moe", "expert": {"ff"}, "router": {"experts", "top"}}``).

Mixer keys: ``attention``: ``heads``, ``kv_heads``, ``dim``, ``vdim``, ``scale``, ``q_temp`` (``coef``,
``every``; absent or null: no query temperature), ``v_mix`` (whether the layer takes part in the mixing of
values: the earliest layer that does is their source); ``general_delta``: ``heads``, ``dim`` (and, optionally, ``decay_rank``: the low
rank of the decay's projection, which a weight file shows by its tensors' shapes); ``hgrn2``: ``heads``, ``dim``,
``vdim``.  Every size and constant comes from there; layers may differ from one another in all of them.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, ClassVar

from .base import ConfigError, ModelConfig, optional, require

MIXER_TYPES = ("attention", "general_delta", "hgrn2")


@dataclass(frozen=True)
class PorovikMixerConfig:
    heads: int
    dim: int
    vdim: int = 0            # attention, hgrn2
    kv_heads: int = 0        # attention
    scale: float = 0.0       # attention
    q_temp_coef: float = 0.0   # attention; every == 0: no query temperature
    q_temp_every: int = 0
    v_mix: bool = False      # attention
    decay_rank: int | None = None  # general_delta: the low rank of the decay's projection; None: as the weight file has it

    @classmethod
    def from_dict(cls, kind: str, raw: Any, where: str) -> "PorovikMixerConfig":
        if not isinstance(raw, dict):
            raise ConfigError(f"config.json: {where}.mixer must be an object")
        heads, dim = require(raw, "heads", int), require(raw, "dim", int)
        if heads <= 0 or dim <= 0:
            raise ConfigError(f"config.json: {where}.mixer: heads and dim must be positive")
        if kind == "general_delta":
            rank = optional(raw, "decay_rank", int, None)
            if rank is not None and rank <= 0:
                raise ConfigError(f"config.json: {where}.mixer.decay_rank must be positive")
            return cls(heads=heads, dim=dim, decay_rank=rank)
        vdim = require(raw, "vdim", int)
        if vdim <= 0:
            raise ConfigError(f"config.json: {where}.mixer.vdim must be positive")
        if kind == "hgrn2":
            return cls(heads=heads, dim=dim, vdim=vdim)
        kv_heads = optional(raw, "kv_heads", int, heads)
        if kv_heads <= 0 or heads % kv_heads:
            raise ConfigError(f"config.json: {where}.mixer: {heads} heads are not a multiple of {kv_heads} kv_heads")
        temp = raw.get("q_temp")
        coef, every = 0.0, 0
        if temp is not None:
            if not isinstance(temp, dict):
                raise ConfigError(f"config.json: {where}.mixer.q_temp must be an object or null")
            coef, every = require(temp, "coef", float), require(temp, "every", int)
            if every <= 0:
                raise ConfigError(f"config.json: {where}.mixer.q_temp.every must be positive")
        return cls(heads=heads, dim=dim, vdim=vdim, kv_heads=kv_heads,
                   scale=optional(raw, "scale", float, float(dim) ** -0.5), q_temp_coef=coef, q_temp_every=every,
                   v_mix=bool(optional(raw, "v_mix", bool, False)))

    def to_dict(self, kind: str) -> dict[str, Any]:
        if kind == "general_delta":
            out = {"heads": self.heads, "dim": self.dim}
            if self.decay_rank is not None:
                out["decay_rank"] = self.decay_rank
            return out
        if kind == "hgrn2":
            return {"heads": self.heads, "dim": self.dim, "vdim": self.vdim}
        out: dict[str, Any] = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim,
                               "scale": self.scale, "v_mix": self.v_mix}
        if self.q_temp_every:
            out["q_temp"] = {"coef": self.q_temp_coef, "every": self.q_temp_every}
        return out


@dataclass(frozen=True)
class PorovikMLPConfig:
    kind: str  # "dense" or "moe"
    ff: int
    experts: int = 0
    top: int = 0

    @classmethod
    def from_dict(cls, raw: Any, where: str) -> "PorovikMLPConfig":
        if not isinstance(raw, dict):
            raise ConfigError(f"config.json: {where}.mlp must be an object or null")
        kind = require(raw, "kind", str)
        if kind == "dense":
            out = cls(kind, require(raw, "ff", int))
        elif kind == "moe":
            expert, router = raw.get("expert"), raw.get("router")
            if not isinstance(expert, dict) or not isinstance(router, dict):
                raise ConfigError(f"config.json: {where}.mlp of kind moe needs expert and router objects")
            out = cls(kind, require(expert, "ff", int), experts=require(router, "experts", int),
                      top=require(router, "top", int))
            if not 0 < out.top <= out.experts:
                raise ConfigError(f"config.json: {where}.mlp.router: top={out.top} of experts={out.experts}")
        else:
            raise ConfigError(f"config.json: {where}.mlp.kind={kind!r}; dense or moe")
        if out.ff <= 0:
            raise ConfigError(f"config.json: {where}.mlp: ff must be positive")
        return out

    def to_dict(self) -> dict[str, Any]:
        if self.kind == "dense":
            return {"kind": "dense", "ff": self.ff}
        return {"kind": "moe", "expert": {"ff": self.ff}, "router": {"experts": self.experts, "top": self.top}}


@dataclass(frozen=True)
class PorovikLayerConfig:
    type: str
    mixer: PorovikMixerConfig
    mlp: PorovikMLPConfig | None


@dataclass(frozen=True)
class PorovikConfig(ModelConfig):
    architecture: ClassVar[str] = "Porovik"

    vocab: int
    width: int
    max_positions: int
    norm_eps: float
    bigram_buckets: int
    bigram_mul_prev: int
    bigram_mul_cur: int
    layers: tuple[PorovikLayerConfig, ...]
    eos_token_id: int | None = None

    def __post_init__(self) -> None:
        if self.vocab <= 0 or self.width <= 0 or self.max_positions <= 0 or not self.layers:
            raise ConfigError("config.json: vocab, width and max_positions must be positive and layers non-empty")
        if self.width % 8:
            raise ConfigError(f"config.json: width={self.width}: the products read rows in 16-byte pieces, so the "
                              "width must be a multiple of 8")
        if self.norm_eps <= 0:
            raise ConfigError("config.json: norm.eps must be positive")
        if self.bigram_buckets <= 0 or self.bigram_mul_prev < 0 or self.bigram_mul_cur < 0:
            raise ConfigError("config.json: embedding.bigram: buckets must be positive, the multipliers not negative")
        if max(self.bigram_mul_prev, self.bigram_mul_cur, self.bigram_buckets) >= 2 ** 31:
            raise ConfigError("config.json: embedding.bigram: buckets and multipliers must fit 32-bit integers")
        mixing = [l.mixer for l in self.layers if l.type == "attention" and l.mixer.v_mix]
        if any(m.kv_heads * m.vdim != mixing[0].kv_heads * mixing[0].vdim for m in mixing):
            raise ConfigError("config.json: layers that mix values (v_mix) must have as many value entries a token "
                              "(kv_heads * vdim) as the first of them")

    @classmethod
    def from_dict(cls, raw: dict[str, Any]) -> "PorovikConfig":
        norm = raw.get("norm")
        if not isinstance(norm, dict):
            raise ConfigError("config.json: norm must be an object with eps")
        emb = raw.get("embedding")
        bigram = emb.get("bigram") if isinstance(emb, dict) else None
        if not isinstance(bigram, dict):
            raise ConfigError("config.json: embedding.bigram must be an object with buckets, mul_prev and mul_cur")
        layers_raw = raw.get("layers")
        if not isinstance(layers_raw, list):
            raise ConfigError("config.json: layers must be a list")
        layers = []
        for i, lr in enumerate(layers_raw):
            where = f"layers[{i}]"
            if not isinstance(lr, dict):
                raise ConfigError(f"config.json: {where} must be an object")
            kind = require(lr, "type", str)
            if kind not in MIXER_TYPES:
                raise ConfigError(f"config.json: {where}.type={kind!r}; the design's mixers: {MIXER_TYPES}")
            mlp = lr.get("mlp")
            layers.append(PorovikLayerConfig(kind, PorovikMixerConfig.from_dict(kind, lr.get("mixer"), where),
                                             None if mlp is None else PorovikMLPConfig.from_dict(mlp, where)))
        return cls(
            vocab=require(raw, "vocab", int), width=require(raw, "width", int),
            max_positions=require(raw, "max_positions", int), norm_eps=require(norm, "eps", float),
            bigram_buckets=require(bigram, "buckets", int), bigram_mul_prev=require(bigram, "mul_prev", int),
            bigram_mul_cur=require(bigram, "mul_cur", int), layers=tuple(layers),
            eos_token_id=optional(raw, "eos_token_id", int, None),
        )

    def to_dict(self) -> dict[str, Any]:
        out: dict[str, Any] = {
            "architecture": self.architecture, "vocab": self.vocab, "width": self.width,
            "max_positions": self.max_positions, "norm": {"eps": self.norm_eps},
            "embedding": {"bigram": {"buckets": self.bigram_buckets, "mul_prev": self.bigram_mul_prev,
                                     "mul_cur": self.bigram_mul_cur}},
            "layers": [{"type": l.type, "mixer": l.mixer.to_dict(l.type), "mlp": None if l.mlp is None else l.mlp.to_dict()}
                       for l in self.layers],
        }
        if self.eos_token_id is not None:
            out["eos_token_id"] = self.eos_token_id
        return out
