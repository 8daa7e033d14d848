"""Lebedra's typed configuration, read from the keys of its own ``config.json``.

Top level: ``vocab``, ``width``, ``residual_mult``, ``norm.eps``, ``token_side.dim`` (absent or
null: no per-layer token input) and ``layers``, a list whose entries give ``type`` (the mixer;
``latent_attention``), the mixer's sizes under ``mixer`` (``heads``, ``dim``, ``rot_dim``,
``vdim``, ``kv_rank``, ``scale``, ``rot.dims``, ``rot.base``) and the feed-forward under ``mlp``:
null for none, ``{"kind": "dense", "ff": n}``, or ``{"kind": "moe", "expert": {"ff", "limit"},
"router": {"experts", "top", "groups": {"count", "keep"}}}``.  Every size and constant comes
from there; layers may differ from one another in all of them.  The design has no position
limit of its own (positions enter through rotations only): ``max_positions``, where a folder
gives it, bounds the sequences the engine plans for, else ``DEFAULT_MAX_POSITIONS``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, ClassVar

from .base import ConfigError, ModelConfig, optional, require

DEFAULT_MAX_POSITIONS = 131072
MIXER_TYPES = ("latent_attention",)


@dataclass(frozen=True)
class LatentMixerConfig:
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    kv_rank: int
    scale: float
    rot_dims: int
    rot_base: float

    @classmethod
    def from_dict(cls, raw: dict[str, Any], where: str) -> "LatentMixerConfig":
        if not isinstance(raw, dict):
            raise ConfigError(f"config.json: {where}.mixer must be an object")
        rot = raw.get("rot")
        if not isinstance(rot, dict):
            raise ConfigError(f"config.json: {where}.mixer.rot must be an object with dims and base")
        dim, rot_dim = require(raw, "dim", int), require(raw, "rot_dim", int)
        out = cls(heads=require(raw, "heads", int), dim=dim, rot_dim=rot_dim, vdim=require(raw, "vdim", int),
                  kv_rank=require(raw, "kv_rank", int),
                  scale=optional(raw, "scale", float, float(dim + rot_dim) ** -0.5),
                  rot_dims=optional(rot, "dims", int, rot_dim), rot_base=require(rot, "base", float))
        for name in ("heads", "dim", "vdim", "kv_rank"):
            if getattr(out, name) <= 0:
                raise ConfigError(f"config.json: {where}.mixer.{name} must be positive")
        if out.rot_dim < 0 or not 0 <= out.rot_dims <= out.rot_dim or out.rot_dims % 2:
            raise ConfigError(f"config.json: {where}.mixer: rot.dims={out.rot_dims} must be even and at most "
                              f"rot_dim={out.rot_dim}")
        if out.rot_base <= 0:
            raise ConfigError(f"config.json: {where}.mixer.rot.base must be positive")
        return out

    def to_dict(self) -> dict[str, Any]:
        return {"heads": self.heads, "dim": self.dim, "rot_dim": self.rot_dim, "vdim": self.vdim,
                "kv_rank": self.kv_rank, "scale": self.scale, "rot": {"dims": self.rot_dims, "base": self.rot_base}}


@dataclass(frozen=True)
class LebedraMLPConfig:
    kind: str                 # "dense" or "moe"
    ff: int
    limit: float = 0.0        # moe: the experts' clamp
    experts: int = 0
    top: int = 0
    group_count: int = 1
    group_keep: int = 1

    @classmethod
    def from_dict(cls, raw: dict[str, Any], where: str) -> "LebedraMLPConfig":
        if not isinstance(raw, dict):
            raise ConfigError(f"config.json: {where}.mlp must be an object or null")
        kind = require(raw, "kind", str)
        if kind == "dense":
            out = cls(kind, require(raw, "ff", int))
        elif kind == "moe":
            expert, router = raw.get("expert"), raw.get("router")
            if not isinstance(expert, dict) or not isinstance(router, dict):
                raise ConfigError(f"config.json: {where}.mlp of kind moe needs expert and router objects")
            groups = router.get("groups") or {}
            if not isinstance(groups, dict):
                raise ConfigError(f"config.json: {where}.mlp.router.groups must be an object")
            out = cls(kind, require(expert, "ff", int), limit=require(expert, "limit", float),
                      experts=require(router, "experts", int), top=require(router, "top", int),
                      group_count=optional(groups, "count", int, 1), group_keep=optional(groups, "keep", int, 1))
            if out.limit <= 0:
                raise ConfigError(f"config.json: {where}.mlp.expert.limit must be positive")
            if not 0 < out.top <= out.experts:
                raise ConfigError(f"config.json: {where}.mlp.router: top={out.top} of experts={out.experts}")
            if out.group_count < 1 or out.experts % out.group_count or not 1 <= out.group_keep <= out.group_count \
                    or out.top > out.group_keep * (out.experts // out.group_count):
                raise ConfigError(f"config.json: {where}.mlp.router.groups: {out.experts} experts in "
                                  f"{out.group_count} groups, {out.group_keep} kept, top {out.top}")
        else:
            raise ConfigError(f"config.json: {where}.mlp.kind={kind!r}; dense or moe")
        if out.ff <= 0:
            raise ConfigError(f"config.json: {where}.mlp: ff must be positive")
        return out

    def to_dict(self) -> dict[str, Any]:
        if self.kind == "dense":
            return {"kind": "dense", "ff": self.ff}
        return {"kind": "moe", "expert": {"ff": self.ff, "limit": self.limit},
                "router": {"experts": self.experts, "top": self.top,
                           "groups": {"count": self.group_count, "keep": self.group_keep}}}


@dataclass(frozen=True)
class LebedraLayerConfig:
    type: str
    mixer: LatentMixerConfig
    mlp: LebedraMLPConfig | None


@dataclass(frozen=True)
class LebedraConfig(ModelConfig):
    architecture: ClassVar[str] = "Lebedra"

    vocab: int
    width: int
    residual_mult: float
    norm_eps: float
    token_side_dim: int | None
    layers: tuple[LebedraLayerConfig, ...]
    max_positions: int = DEFAULT_MAX_POSITIONS
    eos_token_id: int | None = None

    def __post_init__(self) -> None:
        if self.vocab <= 0 or self.width <= 0 or not self.layers:
            raise ConfigError("config.json: vocab and width must be positive and layers non-empty")
        if self.width % 8:
            raise ConfigError(f"config.json: width={self.width}: the products read rows in 16-byte pieces, so the "
                              "width must be a multiple of 8")
        if self.norm_eps <= 0:
            raise ConfigError("config.json: norm.eps must be positive")
        if self.token_side_dim is not None and self.token_side_dim <= 0:
            raise ConfigError("config.json: token_side.dim must be positive")
        if self.max_positions <= 0:
            raise ConfigError("config.json: max_positions must be positive")

    @classmethod
    def from_dict(cls, raw: dict[str, Any]) -> "LebedraConfig":
        norm = raw.get("norm")
        if not isinstance(norm, dict):
            raise ConfigError("config.json: norm must be an object with eps")
        if norm.get("kind", "rms") not in ("rms", "rms_norm"):
            raise ConfigError(f"config.json: norm.kind={norm.get('kind')!r}: the design's norm is the RMS norm")
        side = raw.get("token_side")
        if side is not None and not isinstance(side, dict):
            raise ConfigError("config.json: token_side must be an object or null")
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
            layers.append(LebedraLayerConfig(kind, LatentMixerConfig.from_dict(lr.get("mixer"), where),
                                             None if mlp is None else LebedraMLPConfig.from_dict(mlp, where)))
        return cls(
            vocab=require(raw, "vocab", int), width=require(raw, "width", int),
            residual_mult=optional(raw, "residual_mult", float, 1.0), norm_eps=require(norm, "eps", float),
            token_side_dim=None if side is None else require(side, "dim", int), layers=tuple(layers),
            max_positions=optional(raw, "max_positions", int, DEFAULT_MAX_POSITIONS),
            eos_token_id=optional(raw, "eos_token_id", int, None),
        )

    def to_dict(self) -> dict[str, Any]:
        out: dict[str, Any] = {
            "architecture": self.architecture, "vocab": self.vocab, "width": self.width,
            "residual_mult": self.residual_mult, "norm": {"eps": self.norm_eps},
            "token_side": None if self.token_side_dim is None else {"dim": self.token_side_dim},
            "layers": [{"type": l.type, "mixer": l.mixer.to_dict(), "mlp": None if l.mlp is None else l.mlp.to_dict()}
                       for l in self.layers],
        }
        if self.max_positions != DEFAULT_MAX_POSITIONS:
            out["max_positions"] = self.max_positions
        if self.eos_token_id is not None:
            out["eos_token_id"] = self.eos_token_id
        return out
