"""Configuration of the Zekivik decoder, read from its config.json.

    {"architecture": "Zekivik", "vocab": V, "width": W, "norm": {"eps": e},
     "layers": [{"type": "attention" | "retention", "mixer": {...}, "mlp": {"kind": "dense", "ff": F} | null}, ...],
     "loop": {"start": a, "stop": b, "times": n}}

attention mixer: heads, kv_heads, dim, vdim, conv (taps), scale, rot {dims, base}.
retention mixer: heads, dim, vdim, decay [heads], rot {dims, base}.
Every size and constant comes from the file; nothing has a default but `loop` (absent: no loop).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any

from .base import ConfigError, KeyReader

ATTENTION = "attention"
RETENTION = "retention"


@dataclass(frozen=True)
class Rotation:
    dims: int
    base: float


@dataclass(frozen=True)
class AttentionSizes:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int
    scale: float
    rot: Rotation


@dataclass(frozen=True)
class RetentionSizes:
    heads: int
    dim: int
    vdim: int
    decay: tuple[float, ...]
    rot: Rotation


@dataclass(frozen=True)
class ZekivikLayer:
    type: str
    mixer: Any                 # AttentionSizes | RetentionSizes
    ff: int | None             # width of the dense feed-forward, None: the layer has none


@dataclass(frozen=True)
class Loop:
    start: int
    stop: int
    times: int


@dataclass(frozen=True)
class ZekivikConfig:
    architecture: str
    vocab: int
    width: int
    eps: float
    layers: tuple[ZekivikLayer, ...]
    loop: Loop | None

    @staticmethod
    def from_dict(raw: dict[str, Any]) -> "ZekivikConfig":
        r = KeyReader(raw)
        norm = _obj(r, "norm", "config.json")
        layers = r.array("layers", item=lambda e: isinstance(e, dict))
        if not layers:
            raise ConfigError("config.json: 'layers' is empty")
        out = []
        for i, e in enumerate(layers):
            where = f"config.json: layers[{i}]"
            lr = KeyReader(e, where)
            kind = lr.string("type")
            mr = _obj(lr, "mixer", where)
            if kind == ATTENTION:
                mixer = AttentionSizes(
                    heads=mr.integer("heads", minimum=1), kv_heads=mr.integer("kv_heads", minimum=1),
                    dim=mr.integer("dim", minimum=1), vdim=mr.integer("vdim", minimum=1),
                    conv=mr.integer("conv", minimum=1), scale=mr.number("scale"), rot=_rotation(mr, where))
                if mixer.heads % mixer.kv_heads:
                    raise ConfigError(f"{where}: {mixer.heads} heads do not divide into {mixer.kv_heads} kv_heads")
            elif kind == RETENTION:
                decay = mr.array("decay", item=lambda v: isinstance(v, (int, float)) and not isinstance(v, bool))
                mixer = RetentionSizes(
                    heads=mr.integer("heads", minimum=1), dim=mr.integer("dim", minimum=1),
                    vdim=mr.integer("vdim", minimum=1), decay=tuple(float(v) for v in decay), rot=_rotation(mr, where))
                if len(mixer.decay) != mixer.heads:
                    raise ConfigError(f"{where}: {len(mixer.decay)} decay constants for {mixer.heads} heads")
            else:
                raise ConfigError(f"{where}: unknown layer type '{kind}' ({ATTENTION}, {RETENTION})")
            if mixer.rot.dims > mixer.dim:
                raise ConfigError(f"{where}: rot.dims {mixer.rot.dims} is more than dim {mixer.dim}")
            ff = None
            if lr.has("mlp"):
                fr = _obj(lr, "mlp", where)
                fk = fr.string("kind")
                if fk != "dense":
                    raise ConfigError(f"{where}: unknown mlp kind '{fk}' (dense)")
                ff = fr.integer("ff", minimum=1)
            out.append(ZekivikLayer(kind, mixer, ff))
        loop = None
        if r.has("loop"):
            lp = _obj(r, "loop", "config.json")
            loop = Loop(lp.integer("start", minimum=0), lp.integer("stop", minimum=0), lp.integer("times", minimum=1))
            if not loop.start <= loop.stop <= len(out):
                raise ConfigError(f"config.json: loop {loop.start}..{loop.stop} does not fit {len(out)} layers")
        return ZekivikConfig(
            architecture=r.string("architecture"), vocab=r.integer("vocab", minimum=1),
            width=r.integer("width", minimum=1), eps=norm.number("eps"), layers=tuple(out), loop=loop)

    def runs(self) -> list[tuple[int, int | None]]:
        """(layer, number of the pass it opens or None) in running order: the layers before the loop
        once, the looped range `times` times, the rest once."""
        n = len(self.layers)
        if self.loop is None or self.loop.stop == self.loop.start:
            return [(i, None) for i in range(n)]
        a, b, times = self.loop.start, self.loop.stop, self.loop.times
        order = [(i, None) for i in range(a)]
        for t in range(times):
            order += [(i, t if i == a else None) for i in range(a, b)]
        return order + [(i, None) for i in range(b, n)]


def _obj(r: KeyReader, key: str, where: str) -> KeyReader:
    if not r.has(key):
        raise ConfigError(f"{where}: missing required key '{key}'")
    v = r.raw[key]
    if not isinstance(v, dict):
        raise ConfigError(f"{where}: '{key}' must be an object, got {v!r}")
    r.used.add(key)
    return KeyReader(v, f"{where}: {key}")


def _rotation(mr: KeyReader, where: str) -> Rotation:
    rr = _obj(mr, "rot", where)
    dims = rr.integer("dims", minimum=0)
    if dims % 2:
        raise ConfigError(f"{where}: rot.dims must be even, got {dims}")
    return Rotation(dims, rr.number("base"))
