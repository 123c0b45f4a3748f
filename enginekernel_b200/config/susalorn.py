"""Configuration of the Susalorn decoder (``"architecture": "Susalorn"``).

A Susalorn ``config.json`` is nested: ``vocab``, ``width``, ``norm.eps``, optional ``streams`` (the
number of residual streams; absent: one plain residual stream), a list ``layers`` whose entries name
their mixer (``type``: ``latent_attention`` or ``channel_delta``), the mixer's sizes (``mixer``) and
the feed-forward (``mlp``: ``kind`` ``dense`` or ``moe``, or null for a layer without one), and an
optional ``loop`` (``start``, ``stop``, ``times``): the layers ``start .. stop-1`` run ``times`` times
in a row with the same weights, each pass with cache entries of its own.  Every size and every
constant that can differ between two models of the design is read from the file; nothing is filled in
that the file does not give.
"""

from __future__ import annotations

import dataclasses
from typing import Optional, Tuple, Union

from .base import ConfigError, ModelConfig, _coerce


def _get(raw, name, kind, where, default=dataclasses.MISSING):
    if not isinstance(raw, dict):
        raise ConfigError(f"{where} must be a JSON object, got {type(raw).__name__}")
    if name not in raw or raw[name] is None:
        if default is dataclasses.MISSING:
            raise ConfigError(f"config.json lacks the required key {where}.{name} for Susalorn")
        return default
    return _coerce(f"{where}.{name}", raw[name], kind)


def _positive(obj, names, where):
    for name in names:
        if not getattr(obj, name) > 0:
            raise ConfigError(f"{where}.{name} must be positive, got {getattr(obj, name)}")


@dataclasses.dataclass(frozen=True)
class RotScaling:
    factor: float
    original: float
    fast: float
    slow: float


@dataclasses.dataclass(frozen=True)
class LatentAttentionConfig:
    """``layers[i].mixer`` of a ``latent_attention`` layer."""
    heads: int
    dim: int                 # unrotated query / key size per head
    rot_dim: int             # rotated query / key size per head (the key part is shared by the heads)
    vdim: int
    q_rank: int
    kv_rank: int
    scale: float
    rot_base: float
    rot_dims: int
    rot_scaling: Optional[RotScaling]

    @classmethod
    def from_dict(cls, raw, where):
        rot = raw.get("rot") if isinstance(raw, dict) else None
        if rot is None:
            raise ConfigError(f"config.json lacks the required key {where}.rot for Susalorn")
        sc = rot.get("scaling")
        scaling = None
        if sc is not None:
            w = where + ".rot.scaling"
            scaling = RotScaling(_get(sc, "factor", float, w), _get(sc, "original", float, w),
                                 _get(sc, "fast", float, w), _get(sc, "slow", float, w))
        g = lambda n, k=int: _get(raw, n, k, where)
        return cls(heads=g("heads"), dim=g("dim"), rot_dim=g("rot_dim"), vdim=g("vdim"), q_rank=g("q_rank"),
                   kv_rank=g("kv_rank"), scale=g("scale", float), rot_base=_get(rot, "base", float, where + ".rot"),
                   rot_dims=_get(rot, "dims", int, where + ".rot"), rot_scaling=scaling)

    def to_dict(self):
        rot = {"base": self.rot_base, "dims": self.rot_dims}
        if self.rot_scaling is not None:
            rot["scaling"] = dataclasses.asdict(self.rot_scaling)
        return {"dim": self.dim, "heads": self.heads, "kv_rank": self.kv_rank, "q_rank": self.q_rank, "rot": rot,
                "rot_dim": self.rot_dim, "scale": self.scale, "vdim": self.vdim}

    def validate(self, where):
        _positive(self, ("heads", "dim", "vdim", "q_rank", "kv_rank", "rot_base"), where)
        if self.rot_dim < 0 or self.rot_dims < 0 or self.rot_dims % 2 or self.rot_dims > self.rot_dim:
            raise ConfigError(f"{where}: rot.dims {self.rot_dims} must be even and at most rot_dim {self.rot_dim}")
        if self.rot_scaling is not None:
            _positive(self.rot_scaling, ("factor", "original", "fast", "slow"), where + ".rot.scaling")


@dataclasses.dataclass(frozen=True)
class ChannelDeltaConfig:
    """``layers[i].mixer`` of a ``channel_delta`` layer.  ``rank`` is not a key of the design (the
    low-rank pairs' inner size is a tensor's shape); it is kept for models made from a configuration
    alone, whose random weights need a size."""
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int
    rank: Optional[int] = None

    @classmethod
    def from_dict(cls, raw, where):
        g = lambda n: _get(raw, n, int, where)
        return cls(heads=g("heads"), kv_heads=g("kv_heads"), dim=g("dim"), vdim=g("vdim"), conv=g("conv"),
                   rank=_get(raw, "rank", int, where, None))

    def to_dict(self):
        out = {"conv": self.conv, "dim": self.dim, "heads": self.heads, "kv_heads": self.kv_heads, "vdim": self.vdim}
        if self.rank is not None:
            out["rank"] = self.rank
        return out

    def validate(self, where):
        _positive(self, ("heads", "kv_heads", "dim", "vdim", "conv"), where)
        if self.heads % self.kv_heads:
            raise ConfigError(f"{where}: heads {self.heads} is not a multiple of kv_heads {self.kv_heads}")


@dataclasses.dataclass(frozen=True)
class DenseMlpConfig:
    ff: int
    kind: str = "dense"

    def to_dict(self):
        return {"ff": self.ff, "kind": "dense"}

    def validate(self, where):
        _positive(self, ("ff",), where)


@dataclasses.dataclass(frozen=True)
class MoeMlpConfig:
    ff: int                  # of one expert
    experts: int
    top: int
    scale: float
    groups: int              # 1: no groups
    keep: int
    kind: str = "moe"

    def to_dict(self):
        router = {"experts": self.experts, "scale": self.scale, "top": self.top}
        if self.groups > 1 or self.keep != self.groups:
            router["groups"] = {"count": self.groups, "keep": self.keep}
        return {"expert": {"ff": self.ff}, "kind": "moe", "router": router}

    def validate(self, where):
        _positive(self, ("ff", "experts", "top", "groups", "keep"), where)
        if self.experts % self.groups or self.keep > self.groups:
            raise ConfigError(f"{where}.router: {self.groups} groups must divide {self.experts} experts, and "
                              f"keep {self.keep} cannot exceed them")
        if self.top > self.keep * (self.experts // self.groups):
            raise ConfigError(f"{where}.router: top {self.top} exceeds the experts of the kept groups")


def _mlp_from_dict(raw, where):
    kind = _get(raw, "kind", str, where)
    if kind == "dense":
        return DenseMlpConfig(_get(raw, "ff", int, where))
    if kind == "moe":
        router = raw.get("router")
        w = where + ".router"
        groups = router.get("groups") if isinstance(router, dict) else None
        count = _get(groups, "count", int, w + ".groups") if groups is not None else 1
        keep = _get(groups, "keep", int, w + ".groups") if groups is not None else 1
        return MoeMlpConfig(ff=_get(raw.get("expert"), "ff", int, where + ".expert"),
                            experts=_get(router, "experts", int, w), top=_get(router, "top", int, w),
                            scale=_get(router, "scale", float, w, 1.0), groups=count, keep=keep)
    raise ConfigError(f"{where}.kind {kind!r} is not a Susalorn feed-forward (dense, moe)")


@dataclasses.dataclass(frozen=True)
class SusalornLayer:
    type: str
    mixer: Union[LatentAttentionConfig, ChannelDeltaConfig]
    mlp: Union[None, DenseMlpConfig, MoeMlpConfig]

    MIXERS = {"latent_attention": LatentAttentionConfig, "channel_delta": ChannelDeltaConfig}

    @classmethod
    def from_dict(cls, raw, where):
        kind = _get(raw, "type", str, where)
        if kind not in cls.MIXERS:
            raise ConfigError(f"{where}.type {kind!r} is not a Susalorn mixer ({', '.join(cls.MIXERS)})")
        if raw.get("mixer") is None:
            raise ConfigError(f"config.json lacks the required key {where}.mixer for Susalorn")
        mlp = raw.get("mlp")
        return cls(kind, cls.MIXERS[kind].from_dict(raw["mixer"], where + ".mixer"),
                   None if mlp is None else _mlp_from_dict(mlp, where + ".mlp"))

    def to_dict(self):
        return {"mixer": self.mixer.to_dict(), "mlp": None if self.mlp is None else self.mlp.to_dict(),
                "type": self.type}


@dataclasses.dataclass(frozen=True)
class SusalornLoop:
    start: int
    stop: int
    times: int


@dataclasses.dataclass(frozen=True)
class SusalornConfig(ModelConfig):
    architecture = "Susalorn"

    vocab: int = 0
    width: int = 0
    norm_eps: float = 0.0
    streams: Optional[int] = None
    layers: Tuple[SusalornLayer, ...] = ()
    loop: Optional[SusalornLoop] = None

    @classmethod
    def from_dict(cls, raw: dict) -> "SusalornConfig":
        if not isinstance(raw, dict):
            raise ConfigError(f"config must be a JSON object, got {type(raw).__name__}")
        layers = raw.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError('config.json needs "layers": a list with one entry per layer')
        loop = raw.get("loop")
        if loop is not None:
            loop = SusalornLoop(_get(loop, "start", int, "loop"), _get(loop, "stop", int, "loop"),
                                _get(loop, "times", int, "loop"))
        cfg = cls(vocab=_get(raw, "vocab", int, "config"), width=_get(raw, "width", int, "config"),
                  norm_eps=_get(raw.get("norm"), "eps", float, "norm"),
                  streams=_get(raw, "streams", int, "config", None),
                  layers=tuple(SusalornLayer.from_dict(l, f"layers[{i}]") for i, l in enumerate(layers)),
                  loop=loop)
        cfg.validate()
        return cfg

    def validate(self) -> None:
        for name in ("vocab", "width"):
            if getattr(self, name) <= 0:
                raise ConfigError(f"{name} must be positive, got {getattr(self, name)}")
        if not self.norm_eps > 0:
            raise ConfigError(f"norm.eps must be positive, got {self.norm_eps}")
        if self.streams is not None and not 1 <= self.streams <= 8:
            raise ConfigError(f"streams must be 1 to 8, got {self.streams}")
        if not self.layers:
            raise ConfigError("a Susalorn model needs at least one layer")
        for i, layer in enumerate(self.layers):
            layer.mixer.validate(f"layers[{i}].mixer")
            if layer.mlp is not None:
                layer.mlp.validate(f"layers[{i}].mlp")
        if self.loop is not None:
            lp = self.loop
            if not (0 <= lp.start <= lp.stop <= len(self.layers)):
                raise ConfigError(f"loop {lp.start}..{lp.stop} does not lie within the {len(self.layers)} layers")
            if lp.times < 1:
                raise ConfigError(f"loop.times must be at least 1, got {lp.times}")

    def to_dict(self) -> dict:
        out = {"architecture": self.architecture, "layers": [l.to_dict() for l in self.layers],
               "norm": {"eps": self.norm_eps}, "vocab": self.vocab, "width": self.width}
        if self.streams is not None:
            out["streams"] = self.streams
        if self.loop is not None:
            out["loop"] = {"start": self.loop.start, "stop": self.loop.stop, "times": self.loop.times}
        return out

    def runs(self):
        """Layer indices in the order they run: before the loop once, the loop's layers ``times``
        times, the rest once."""
        n = len(self.layers)
        lp = self.loop or SusalornLoop(0, 0, 1)
        order = list(range(lp.start))
        for _ in range(lp.times):
            order += list(range(lp.start, lp.stop))
        return order + list(range(lp.stop, n))
