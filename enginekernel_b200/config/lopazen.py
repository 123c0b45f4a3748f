"""Configuration of the Lopazen decoder (``"architecture": "Lopazen"``).

A Lopazen ``config.json`` is nested: ``vocab``, ``width``, ``embedding.scale``, ``norm.eps``, a
list ``layers`` whose entries name their mixer (``type``), the mixer's sizes (``mixer``) and the
feed-forward (``mlp``, or null for a layer without one), and an optional ``loop`` (``start``,
``stop``, ``times``): the layers ``start .. stop-1`` run ``times`` times in a row with the same
weights.  Every size and every constant that can differ between two models of the design is read
from the file; nothing is filled in that the file does not give.
"""

from __future__ import annotations

import dataclasses
from typing import Optional, Tuple

from .base import ConfigError, ModelConfig, _coerce


def _get(raw, name, kind, where, default=dataclasses.MISSING):
    if not isinstance(raw, dict):
        raise ConfigError(f"{where} must be a JSON object, got {type(raw).__name__}")
    if name not in raw or raw[name] is None:
        if default is dataclasses.MISSING:
            raise ConfigError(f"config.json lacks the required key {where}.{name} for Lopazen")
        return default
    return _coerce(f"{where}.{name}", raw[name], kind)


@dataclasses.dataclass(frozen=True)
class LopazenAttention:
    """Sizes and constants of one attention mixer (``layers[i].mixer``)."""
    heads: int
    kv_heads: int
    dim: int                 # per-head query / key size
    vdim: int                # per-head value size
    scale: float             # factor on q.k
    q_temp_coef: float       # 0: no query temperature
    q_temp_every: int

    @classmethod
    def from_dict(cls, raw, where):
        temp = raw.get("q_temp") if isinstance(raw, dict) else None
        coef, every = 0.0, 1
        if temp is not None:
            coef = _get(temp, "coef", float, where + ".q_temp")
            every = _get(temp, "every", int, where + ".q_temp")
        return cls(heads=_get(raw, "heads", int, where), kv_heads=_get(raw, "kv_heads", int, where),
                   dim=_get(raw, "dim", int, where), vdim=_get(raw, "vdim", int, where),
                   scale=_get(raw, "scale", float, where), q_temp_coef=coef, q_temp_every=every)

    def to_dict(self):
        return {"dim": self.dim, "heads": self.heads, "kv_heads": self.kv_heads,
                "q_temp": {"coef": self.q_temp_coef, "every": self.q_temp_every},
                "scale": self.scale, "vdim": self.vdim}

    def validate(self, where):
        for name in ("heads", "kv_heads", "dim", "vdim", "q_temp_every"):
            if getattr(self, name) <= 0:
                raise ConfigError(f"{where}.{name} must be positive, got {getattr(self, name)}")
        if self.heads % self.kv_heads:
            raise ConfigError(f"{where}: heads {self.heads} is not a multiple of kv_heads {self.kv_heads}")
        if self.vdim != self.dim:
            raise ConfigError(f"{where}: the values are the keys as projected, so vdim {self.vdim} "
                              f"must equal dim {self.dim}")


@dataclasses.dataclass(frozen=True)
class LopazenMlp:
    kind: str                # "dense"
    ff: int

    @classmethod
    def from_dict(cls, raw, where):
        return cls(kind=_get(raw, "kind", str, where), ff=_get(raw, "ff", int, where))

    def to_dict(self):
        return {"ff": self.ff, "kind": self.kind}

    def validate(self, where):
        if self.kind != "dense":
            raise ConfigError(f"{where}.kind {self.kind!r} is not a Lopazen feed-forward (dense)")
        if self.ff <= 0:
            raise ConfigError(f"{where}.ff must be positive, got {self.ff}")


@dataclasses.dataclass(frozen=True)
class LopazenLayer:
    type: str                # which mixer: "attention"
    mixer: LopazenAttention
    mlp: Optional[LopazenMlp]

    @classmethod
    def from_dict(cls, raw, where):
        kind = _get(raw, "type", str, where)
        if kind != "attention":
            raise ConfigError(f"{where}.type {kind!r} is not a Lopazen mixer (attention)")
        mixer = raw.get("mixer")
        if mixer is None:
            raise ConfigError(f"config.json lacks the required key {where}.mixer for Lopazen")
        mlp = raw.get("mlp")
        return cls(kind, LopazenAttention.from_dict(mixer, where + ".mixer"),
                   None if mlp is None else LopazenMlp.from_dict(mlp, where + ".mlp"))

    def to_dict(self):
        return {"mixer": self.mixer.to_dict(), "mlp": None if self.mlp is None else self.mlp.to_dict(),
                "type": self.type}


@dataclasses.dataclass(frozen=True)
class LopazenLoop:
    start: int
    stop: int
    times: int


@dataclasses.dataclass(frozen=True)
class LopazenConfig(ModelConfig):
    architecture = "Lopazen"

    vocab: int = 0
    width: int = 0
    embedding_scale: float = 1.0
    norm_eps: float = 0.0
    layers: Tuple[LopazenLayer, ...] = ()
    loop: Optional[LopazenLoop] = None

    @classmethod
    def from_dict(cls, raw: dict) -> "LopazenConfig":
        if not isinstance(raw, dict):
            raise ConfigError(f"config must be a JSON object, got {type(raw).__name__}")
        layers = raw.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError('config.json needs "layers": a list with one entry per layer')
        loop = raw.get("loop")
        if loop is not None:
            loop = LopazenLoop(_get(loop, "start", int, "loop"), _get(loop, "stop", int, "loop"),
                               _get(loop, "times", int, "loop"))
        cfg = cls(vocab=_get(raw, "vocab", int, "config"), width=_get(raw, "width", int, "config"),
                  embedding_scale=_get(raw.get("embedding"), "scale", float, "embedding"),
                  norm_eps=_get(raw.get("norm"), "eps", float, "norm"),
                  layers=tuple(LopazenLayer.from_dict(l, f"layers[{i}]") for i, l in enumerate(layers)),
                  loop=loop)
        cfg.validate()
        return cfg

    def validate(self) -> None:
        for name in ("vocab", "width"):
            if getattr(self, name) <= 0:
                raise ConfigError(f"{name} must be positive, got {getattr(self, name)}")
        if not self.norm_eps > 0:
            raise ConfigError(f"norm.eps must be positive, got {self.norm_eps}")
        if not self.layers:
            raise ConfigError("a Lopazen model needs at least one layer")
        for i, layer in enumerate(self.layers):
            layer.mixer.validate(f"layers[{i}].mixer")
            if layer.mlp is not None:
                layer.mlp.validate(f"layers[{i}].mlp")
        if self.loop is not None:
            lp = self.loop
            if not (0 <= lp.start <= lp.stop <= len(self.layers)):
                raise ConfigError(f"loop {lp.start}..{lp.stop} does not lie within the "
                                  f"{len(self.layers)} layers")
            if lp.times < 1:
                raise ConfigError(f"loop.times must be at least 1, got {lp.times}")

    def to_dict(self) -> dict:
        out = {"architecture": self.architecture, "embedding": {"scale": self.embedding_scale},
               "layers": [l.to_dict() for l in self.layers], "norm": {"eps": self.norm_eps},
               "vocab": self.vocab, "width": self.width}
        if self.loop is not None:
            out["loop"] = {"start": self.loop.start, "stop": self.loop.stop, "times": self.loop.times}
        return out

    def runs(self):
        """The order in which layers run: (layer index, whether a further pass of the loop starts
        here).  Layers before the loop once, the loop's layers ``times`` times, the rest once."""
        n = len(self.layers)
        lp = self.loop or LopazenLoop(0, 0, 1)
        order = [(i, False) for i in range(lp.start)]
        for p in range(lp.times):
            order += [(i, p > 0 and i == lp.start) for i in range(lp.start, lp.stop)]
        order += [(i, False) for i in range(lp.stop, n)]
        return order
