"""Typed configuration of the Puladra design, read from its own ``config.json`` keys.

The file lists the layers one by one: each entry names its mixer (``type``: ``gla`` or
``parallel``) with the mixer's sizes and constants (``mixer``) and its feed-forward (``mlp``, or
null for none).  ``loop`` says which run of layers is repeated with the same weights (a learned
vector per pass is added to the stream before each pass), ``token_side`` gives the width of the
per-layer token input, ``logit_scale`` multiplies the logits of the tied output head.  Every size
and constant that can differ between two models of the design is a field here; nothing is
assumed equal between layers.
"""

from __future__ import annotations

import copy
import dataclasses
from dataclasses import dataclass, field
from typing import Any, Mapping

from .model_config import ConfigError, _require


def _positive_int(where: str, raw: Mapping[str, Any], key: str) -> int:
    if key not in raw or raw[key] is None:
        raise ConfigError(f"{where}: missing key {key!r}")
    value = raw[key]
    if int(value) != value or int(value) < 1:
        raise ConfigError(f"{where}: {key} must be a positive integer, got {value!r}")
    return int(value)


@dataclass(frozen=True)
class RotationConfig:
    """Pairs (i, i + dims / 2) of the first ``dims`` elements of a head turn by p * base^(-2i / dims)."""

    dims: int
    base: float

    @classmethod
    def from_raw(cls, where: str, raw: Mapping[str, Any] | None, head_dim: int) -> "RotationConfig | None":
        if not raw:
            return None
        cfg = cls(dims=_positive_int(where + ".rot", raw, "dims"), base=float(_require(raw, "base")))
        if cfg.dims % 2 or cfg.dims > head_dim:
            raise ConfigError(f"{where}: rot.dims={cfg.dims} must be even and at most dim={head_dim}")
        if not cfg.base > 0:
            raise ConfigError(f"{where}: rot.base must be positive")
        return cfg

    def to_raw(self) -> dict[str, Any]:
        return dict(base=self.base, dims=self.dims)


@dataclass(frozen=True)
class GlaConfig:
    """Gated linear attention: a decay per key channel and token, sigmoid(z)^(1 / tau)."""

    heads: int
    dim: int
    vdim: int
    tau: float
    # rows of the decay's low-rank matrix; config.json does not say: 0 until the stored tensor's
    # shape has been read (PuladraConfig.with_tensor_shapes)
    decay_rank: int = 0

    @classmethod
    def from_raw(cls, where: str, raw: Mapping[str, Any]) -> "GlaConfig":
        cfg = cls(heads=_positive_int(where, raw, "heads"), dim=_positive_int(where, raw, "dim"),
                  vdim=_positive_int(where, raw, "vdim"), tau=float(_require(raw, "tau")),
                  decay_rank=int(raw.get("decay_rank") or 0))  # an optional key: a model that is yet to be written
        if not cfg.tau > 0:
            raise ConfigError(f"{where}: tau must be positive")
        return cfg

    def to_raw(self) -> dict[str, Any]:
        return dict(heads=self.heads, dim=self.dim, vdim=self.vdim, tau=self.tau)


@dataclass(frozen=True)
class WindowAttentionConfig:
    """Softmax attention with grouped key/value heads, a short convolution on q, k and v, a
    rotation of q and k and a sliding window."""

    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    conv: int  # taps of the short convolution; 0: none
    rot: RotationConfig | None
    window: int | None  # position i sees j with 0 <= i - j < window; None: every j <= i

    @classmethod
    def from_raw(cls, where: str, raw: Mapping[str, Any]) -> "WindowAttentionConfig":
        dim = _positive_int(where, raw, "dim")
        mask = raw.get("mask") or {}
        cfg = cls(heads=_positive_int(where, raw, "heads"), kv_heads=_positive_int(where, raw, "kv_heads"), dim=dim,
                  vdim=_positive_int(where, raw, "vdim"), scale=float(_require(raw, "scale")),
                  conv=int(raw.get("conv") or 0), rot=RotationConfig.from_raw(where, raw.get("rot"), dim),
                  window=int(mask["size"]) if mask.get("size") else None)
        if cfg.heads % cfg.kv_heads:
            raise ConfigError(f"{where}: heads={cfg.heads} is no multiple of kv_heads={cfg.kv_heads}")
        if cfg.conv < 0 or (cfg.window is not None and cfg.window < 1):
            raise ConfigError(f"{where}: conv must not be negative and mask.size must be positive")
        return cfg

    def to_raw(self) -> dict[str, Any]:
        out: dict[str, Any] = dict(heads=self.heads, kv_heads=self.kv_heads, dim=self.dim, vdim=self.vdim,
                                   scale=self.scale)
        if self.conv:
            out["conv"] = self.conv
        if self.rot is not None:
            out["rot"] = self.rot.to_raw()
        if self.window is not None:
            out["mask"] = dict(size=self.window)
        return out


@dataclass(frozen=True)
class RetentionConfig:
    """Linear attention with one fixed decay per head, no softmax and no denominator."""

    heads: int
    dim: int
    vdim: int
    decay: tuple[float, ...]
    rot: RotationConfig | None

    @classmethod
    def from_raw(cls, where: str, raw: Mapping[str, Any]) -> "RetentionConfig":
        dim = _positive_int(where, raw, "dim")
        cfg = cls(heads=_positive_int(where, raw, "heads"), dim=dim, vdim=_positive_int(where, raw, "vdim"),
                  decay=tuple(float(d) for d in _require(raw, "decay")),
                  rot=RotationConfig.from_raw(where, raw.get("rot"), dim))
        if len(cfg.decay) != cfg.heads:
            raise ConfigError(f"{where}: {len(cfg.decay)} decays for {cfg.heads} heads")
        return cfg

    def to_raw(self) -> dict[str, Any]:
        out: dict[str, Any] = dict(heads=self.heads, dim=self.dim, vdim=self.vdim, decay=list(self.decay))
        if self.rot is not None:
            out["rot"] = self.rot.to_raw()
        return out


@dataclass(frozen=True)
class ParallelConfig:
    """Two mixers side by side on the same input; the result is a weighted sum of the two."""

    left: WindowAttentionConfig
    right: RetentionConfig
    left_scale: float
    right_scale: float

    @classmethod
    def from_raw(cls, where: str, raw: Mapping[str, Any]) -> "ParallelConfig":
        return cls(left=WindowAttentionConfig.from_raw(where + ".left", _require(raw, "left")),
                   right=RetentionConfig.from_raw(where + ".right", _require(raw, "right")),
                   left_scale=float(raw.get("left_scale", 1.0)), right_scale=float(raw.get("right_scale", 1.0)))

    def to_raw(self) -> dict[str, Any]:
        return dict(left=self.left.to_raw(), right=self.right.to_raw(), left_scale=self.left_scale,
                    right_scale=self.right_scale)


@dataclass(frozen=True)
class MoeConfig:
    """``experts`` squared-ReLU layers of width ``ff`` of which a token uses ``top`` (weights: the
    softmax over the chosen router logits), and an optional shared one of width ``shared_ff``
    that runs for every token behind a sigmoid gate."""

    experts: int
    top: int
    ff: int
    shared_ff: int = 0

    @classmethod
    def from_raw(cls, where: str, raw: Mapping[str, Any]) -> "MoeConfig":
        kind = _require(raw, "kind")
        if kind != "moe":
            raise ConfigError(f"{where}: unknown feed-forward kind {kind!r}")
        router = _require(raw, "router")
        shared = raw.get("shared") or {}
        cfg = cls(experts=_positive_int(where + ".router", router, "experts"),
                  top=_positive_int(where + ".router", router, "top"),
                  ff=_positive_int(where + ".expert", _require(raw, "expert"), "ff"),
                  shared_ff=_positive_int(where + ".shared", shared, "ff") if shared else 0)
        if cfg.top > cfg.experts:
            raise ConfigError(f"{where}: top={cfg.top} exceeds experts={cfg.experts}")
        return cfg

    def to_raw(self) -> dict[str, Any]:
        out: dict[str, Any] = dict(kind="moe", router=dict(experts=self.experts, top=self.top),
                                   expert=dict(ff=self.ff))
        if self.shared_ff:
            out["shared"] = dict(ff=self.shared_ff)
        return out


@dataclass(frozen=True)
class PuladraLayerConfig:
    type: str
    mixer: GlaConfig | ParallelConfig
    mlp: MoeConfig | None


MIXER_CONFIGS = {"gla": GlaConfig, "parallel": ParallelConfig}


@dataclass(frozen=True)
class PuladraConfig:
    vocab: int
    width: int
    norm_eps: float
    layers: tuple[PuladraLayerConfig, ...]
    logit_scale: float = 1.0
    side_dim: int = 0  # width of the per-layer token input; 0: the model has none
    # layers loop_start .. loop_stop - 1 run loop_times times in a row with the same weights;
    # loop_times == 0: the model has no loop (and no vector per pass)
    loop_start: int = 0
    loop_stop: int = 0
    loop_times: int = 0
    extra: dict = field(default_factory=dict, compare=False, repr=False)

    architecture = "Puladra"

    def __post_init__(self) -> None:
        if self.vocab < 1 or self.width < 1 or not self.layers:
            raise ConfigError("vocab, width and the number of layers must be positive")
        if not self.norm_eps > 0:
            raise ConfigError(f"norm.eps must be positive, got {self.norm_eps!r}")
        if self.loop_times < 0 or self.side_dim < 0:
            raise ConfigError("loop.times and token_side.dim must not be negative")
        if self.loop_times and not 0 <= self.loop_start < self.loop_stop <= len(self.layers):
            raise ConfigError(f"loop {self.loop_start}..{self.loop_stop} does not fit {len(self.layers)} layers")

    @classmethod
    def from_hf_config(cls, raw: Mapping[str, Any]) -> "PuladraConfig":
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
            layers.append(PuladraLayerConfig(kind, mixer, MoeConfig.from_raw(f"layer {i} mlp", mlp) if mlp else None))
        loop = raw.get("loop") or {}
        side = raw.get("token_side") or {}
        return cls(vocab=int(_require(raw, "vocab")), width=int(_require(raw, "width")),
                   norm_eps=float(_require(_require(raw, "norm"), "eps")), layers=tuple(layers),
                   logit_scale=float(raw.get("logit_scale", 1.0)), side_dim=int(side.get("dim") or 0),
                   loop_start=int(loop.get("start", 0)), loop_stop=int(loop.get("stop", 0)),
                   loop_times=int(loop.get("times", 1)) if loop else 0)

    def to_hf_config(self) -> dict[str, Any]:
        """The ``config.json`` dictionary that :meth:`from_hf_config` reads back."""
        out: dict[str, Any] = dict(architecture=self.architecture, vocab=self.vocab, width=self.width,
                                   norm=dict(eps=self.norm_eps), logit_scale=self.logit_scale)
        out["layers"] = [dict(type=l.type, mixer=l.mixer.to_raw(), mlp=l.mlp.to_raw() if l.mlp else None)
                         for l in self.layers]
        if self.loop_times:
            out["loop"] = dict(start=self.loop_start, stop=self.loop_stop, times=self.loop_times)
        if self.side_dim:
            out["token_side"] = dict(dim=self.side_dim)
        return copy.deepcopy(out)

    def with_tensor_shapes(self, shape_of) -> "PuladraConfig":
        """The sizes that only the stored tensors give: ``shape_of(name)`` is a tensor's shape.  The
        decay of a ``gla`` mixer goes through a low-rank product whose rank is the row count of
        ``l<i>.mix.a1``."""
        layers = []
        for i, layer in enumerate(self.layers):
            if isinstance(layer.mixer, GlaConfig) and not layer.mixer.decay_rank:
                rank = int(shape_of(f"l{i}.mix.a1")[0])
                layer = dataclasses.replace(layer, mixer=dataclasses.replace(layer.mixer, decay_rank=rank))
            layers.append(layer)
        return dataclasses.replace(self, layers=tuple(layers))

    def run_order(self) -> list[tuple[int, int | None]]:
        """``(layer, number of the loop pass that this run starts, or None)`` for every layer run:
        the looped layers appear ``loop_times`` times, and the first layer of each pass (the first
        pass too) is marked with the pass's number."""
        n = len(self.layers)
        if not self.loop_times:
            return [(i, None) for i in range(n)]
        order: list[tuple[int, int | None]] = [(i, None) for i in range(self.loop_start)]
        for rep in range(self.loop_times):
            order += [(i, rep if i == self.loop_start else None) for i in range(self.loop_start, self.loop_stop)]
        return order + [(i, None) for i in range(self.loop_stop, n)]
