"""Typed configuration of the Logesun design, read from its own ``config.json`` keys.

The file lists the layers one by one: each entry names its mixer (``type``) with the mixer's
sizes and constants (``mixer``) and its feed-forward (``mlp``, or null for none).  ``loop`` says
which run of layers is repeated with the same weights.  Every size and constant that can differ
between two models of the design is a field here; nothing is assumed equal between layers.
"""

from __future__ import annotations

import copy
from dataclasses import dataclass, field
from typing import Any, Mapping

from .model_config import ConfigError, _require


def _positive_int(where: str, raw: Mapping[str, Any], key: str) -> int:
    value = _require(raw, key) if key in raw else None
    if value is None:
        raise ConfigError(f"{where}: missing key {key!r}")
    if int(value) != value or int(value) < 1:
        raise ConfigError(f"{where}: {key} must be a positive integer, got {value!r}")
    return int(value)


@dataclass(frozen=True)
class LatentAttentionConfig:
    """Sizes and constants of one ``latent_attention`` mixer."""

    heads: int
    dim: int  # unrotated query/key dimensions per head
    rot_dim: int  # rotated query/key dimensions per head (one key part shared by all heads)
    vdim: int
    q_rank: int
    kv_rank: int
    scale: float
    rot_dims: int  # how many of the rotated part's dimensions turn (pairs 2i, 2i + 1)
    rot_base: float
    window: int | None  # the query at position p reads positions max(0, p - window + 1) .. p; None: all from 0

    @classmethod
    def from_raw(cls, where: str, raw: Mapping[str, Any]) -> "LatentAttentionConfig":
        rot = raw.get("rot") or {}
        mask = raw.get("mask") or {}
        rot_dim = _positive_int(where, raw, "rot_dim")
        cfg = cls(
            heads=_positive_int(where, raw, "heads"), dim=_positive_int(where, raw, "dim"), rot_dim=rot_dim,
            vdim=_positive_int(where, raw, "vdim"), q_rank=_positive_int(where, raw, "q_rank"),
            kv_rank=_positive_int(where, raw, "kv_rank"), scale=float(_require(raw, "scale")),
            rot_dims=int(rot.get("dims", rot_dim)), rot_base=float(rot.get("base", 10000.0)),
            window=int(mask["size"]) if mask.get("size") else None)
        if cfg.rot_dims < 2 or cfg.rot_dims % 2 or cfg.rot_dims > cfg.rot_dim:
            raise ConfigError(f"{where}: rot.dims={cfg.rot_dims} must be even and at most rot_dim={cfg.rot_dim}")
        if not cfg.rot_base > 0 or not cfg.scale > 0:
            raise ConfigError(f"{where}: rot.base and scale must be positive")
        if cfg.window is not None and cfg.window < 1:
            raise ConfigError(f"{where}: mask.size must be positive")
        return cfg

    def to_raw(self) -> dict[str, Any]:
        out = dict(heads=self.heads, dim=self.dim, rot_dim=self.rot_dim, vdim=self.vdim, q_rank=self.q_rank,
                   kv_rank=self.kv_rank, scale=self.scale, rot=dict(base=self.rot_base, dims=self.rot_dims))
        if self.window is not None:
            out["mask"] = dict(size=self.window)
        return out


@dataclass(frozen=True)
class ExpertConfig:
    ff: int
    limit: float

    @classmethod
    def from_raw(cls, where: str, raw: Mapping[str, Any]) -> "ExpertConfig":
        cfg = cls(ff=_positive_int(where, raw, "ff"), limit=float(_require(raw, "limit")))
        if not cfg.limit > 0:
            raise ConfigError(f"{where}: limit must be positive")
        return cfg


@dataclass(frozen=True)
class FeedForwardConfig:
    """``kind`` dense: one SwiGLU layer of width ``ff``.  ``kind`` moe: ``experts`` clamped gated
    layers of which a token uses ``top``, and an optional shared one."""

    kind: str
    ff: int = 0
    experts: int = 0
    top: int = 0
    expert: ExpertConfig | None = None
    shared: ExpertConfig | None = None

    @classmethod
    def from_raw(cls, where: str, raw: Mapping[str, Any]) -> "FeedForwardConfig":
        kind = _require(raw, "kind")
        if kind == "dense":
            return cls(kind="dense", ff=_positive_int(where, raw, "ff"))
        if kind == "moe":
            router = _require(raw, "router")
            cfg = cls(kind="moe", experts=_positive_int(where + ".router", router, "experts"),
                      top=_positive_int(where + ".router", router, "top"),
                      expert=ExpertConfig.from_raw(where + ".expert", _require(raw, "expert")),
                      shared=ExpertConfig.from_raw(where + ".shared", raw["shared"]) if raw.get("shared") else None)
            if cfg.top > cfg.experts:
                raise ConfigError(f"{where}: top={cfg.top} exceeds experts={cfg.experts}")
            return cfg
        raise ConfigError(f"{where}: unknown feed-forward kind {kind!r}")

    def to_raw(self) -> dict[str, Any]:
        if self.kind == "dense":
            return dict(kind="dense", ff=self.ff)
        out: dict[str, Any] = dict(kind="moe", router=dict(experts=self.experts, top=self.top),
                                   expert=dict(ff=self.expert.ff, limit=self.expert.limit))
        if self.shared is not None:
            out["shared"] = dict(ff=self.shared.ff, limit=self.shared.limit)
        return out


@dataclass(frozen=True)
class LogesunLayerConfig:
    type: str
    mixer: LatentAttentionConfig
    mlp: FeedForwardConfig | None


MIXER_CONFIGS = {"latent_attention": LatentAttentionConfig}


@dataclass(frozen=True)
class LogesunConfig:
    vocab: int
    width: int
    norm_eps: float
    layers: tuple[LogesunLayerConfig, ...]
    # layers loop_start .. loop_stop - 1 run loop_times times in a row with the same weights
    loop_start: int = 0
    loop_stop: int = 0
    loop_times: int = 1
    extra: dict = field(default_factory=dict, compare=False, repr=False)

    architecture = "Logesun"

    def __post_init__(self) -> None:
        if self.vocab < 1 or self.width < 1 or not self.layers:
            raise ConfigError("vocab, width and the number of layers must be positive")
        if not self.norm_eps > 0:
            raise ConfigError(f"norm.eps must be positive, got {self.norm_eps!r}")
        if self.loop_times < 1:
            raise ConfigError("loop.times must be at least 1")
        if self.loop_times > 1 and not 0 <= self.loop_start <= self.loop_stop <= len(self.layers):
            raise ConfigError(f"loop {self.loop_start}..{self.loop_stop} does not fit {len(self.layers)} layers")

    @classmethod
    def from_hf_config(cls, raw: Mapping[str, Any]) -> "LogesunConfig":
        names = [raw.get("architecture"), *(raw.get("architectures") or [])]
        if cls.architecture not in names:
            raise ConfigError(f"unsupported architecture: {names}")
        layers = []
        for i, entry in enumerate(_require(raw, "layers")):
            kind = _require(entry, "type")
            if kind not in MIXER_CONFIGS:
                raise ConfigError(f"layer {i}: unknown mixer type {kind!r} (known: {sorted(MIXER_CONFIGS)})")
            mixer = MIXER_CONFIGS[kind].from_raw(f"layer {i} mixer", _require(entry, "mixer"))
            mlp = entry.get("mlp")
            layers.append(LogesunLayerConfig(kind, mixer,
                                             FeedForwardConfig.from_raw(f"layer {i} mlp", mlp) if mlp else None))
        loop = raw.get("loop") or {}
        return cls(vocab=int(_require(raw, "vocab")), width=int(_require(raw, "width")),
                   norm_eps=float(_require(_require(raw, "norm"), "eps")), layers=tuple(layers),
                   loop_start=int(loop.get("start", 0)), loop_stop=int(loop.get("stop", 0)),
                   loop_times=int(loop.get("times", 1)))

    def to_hf_config(self) -> dict[str, Any]:
        """The ``config.json`` dictionary that :meth:`from_hf_config` reads back."""
        out: dict[str, Any] = dict(architecture=self.architecture, vocab=self.vocab, width=self.width,
                                   norm=dict(eps=self.norm_eps))
        out["layers"] = [dict(type=l.type, mixer=l.mixer.to_raw(), mlp=l.mlp.to_raw() if l.mlp else None)
                         for l in self.layers]
        if self.loop_times > 1:
            out["loop"] = dict(start=self.loop_start, stop=self.loop_stop, times=self.loop_times)
        return copy.deepcopy(out)

    def run_order(self) -> list[tuple[int, bool]]:
        """``(layer, embedding added right before it)`` for every layer run: the looped layers
        appear ``loop_times`` times, and every pass but the first starts from x + embedding."""
        n = len(self.layers)
        if self.loop_times <= 1 or self.loop_start >= self.loop_stop:  # nothing is repeated
            return [(i, False) for i in range(n)]
        order = [(i, False) for i in range(self.loop_start)]
        for rep in range(self.loop_times):
            order += [(i, rep > 0 and i == self.loop_start) for i in range(self.loop_start, self.loop_stop)]
        return order + [(i, False) for i in range(self.loop_stop, n)]
