"""Configuration of the Lenesun decoder, read from its config.json.

    {"architecture": "Lenesun", "vocab": V, "width": W, "norm": {"eps": e}, "residual_mult": m,
     "embedding": {"scale": s},
     "layers": [{"type": "latent_attention", "mixer": {...}, "mlp": {...} | null}, ...]}

latent_attention mixer: heads, dim (unrotated query/key numbers per head), rot_dim (rotated ones),
vdim, q_rank, kv_rank, scale, rot {dims, base}, and optionally kv_from (the layer whose cached rows
this layer reads instead of projecting its own).
mlp: {"kind": "moe", "router": {"experts": E, "top": k}, "expert": {"ff": F, "limit": L}}.
Every size and constant comes from the file; nothing has a default.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any

from .base import ConfigError, KeyReader
from .zekivik import Rotation, _obj, _rotation

LATENT_ATTENTION = "latent_attention"


@dataclass(frozen=True)
class LatentAttentionSizes:
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    q_rank: int
    kv_rank: int
    scale: float
    rot: Rotation
    kv_from: int | None


@dataclass(frozen=True)
class MoeSizes:
    experts: int
    top: int
    ff: int
    limit: float


@dataclass(frozen=True)
class LenesunLayer:
    type: str
    mixer: LatentAttentionSizes
    mlp: MoeSizes | None


@dataclass(frozen=True)
class LenesunConfig:
    architecture: str
    vocab: int
    width: int
    eps: float
    residual_mult: float
    embedding_scale: float
    layers: tuple[LenesunLayer, ...]

    @staticmethod
    def from_dict(raw: dict[str, Any]) -> "LenesunConfig":
        r = KeyReader(raw)
        norm = _obj(r, "norm", "config.json")
        emb = _obj(r, "embedding", "config.json")
        layers = r.array("layers", item=lambda e: isinstance(e, dict))
        if not layers:
            raise ConfigError("config.json: 'layers' is empty")
        out: list[LenesunLayer] = []
        for i, e in enumerate(layers):
            where = f"config.json: layers[{i}]"
            lr = KeyReader(e, where)
            kind = lr.string("type")
            if kind != LATENT_ATTENTION:
                raise ConfigError(f"{where}: unknown layer type '{kind}' ({LATENT_ATTENTION})")
            mr = _obj(lr, "mixer", where)
            m = LatentAttentionSizes(
                heads=mr.integer("heads", minimum=1), dim=mr.integer("dim", minimum=1),
                rot_dim=mr.integer("rot_dim", minimum=0), vdim=mr.integer("vdim", minimum=1),
                q_rank=mr.integer("q_rank", minimum=1), kv_rank=mr.integer("kv_rank", minimum=1),
                scale=mr.number("scale"), rot=_rotation(mr, where),
                kv_from=mr.integer("kv_from", minimum=0) if mr.has("kv_from") else None)
            if m.rot.dims > m.rot_dim:
                raise ConfigError(f"{where}: rot.dims {m.rot.dims} is more than rot_dim {m.rot_dim}")
            if m.kv_from is not None:
                if m.kv_from >= i:
                    raise ConfigError(f"{where}: kv_from {m.kv_from} must name an earlier layer")
                src = out[m.kv_from].mixer
                if src.kv_from is not None:
                    raise ConfigError(f"{where}: kv_from {m.kv_from} names a layer that caches nothing of its own")
                if (src.kv_rank, src.rot_dim, src.rot) != (m.kv_rank, m.rot_dim, m.rot):
                    raise ConfigError(f"{where}: kv_rank, rot_dim and rot must equal those of layer {m.kv_from}")
            mlp = None
            if lr.has("mlp"):
                fr = _obj(lr, "mlp", where)
                fk = fr.string("kind")
                if fk != "moe":
                    raise ConfigError(f"{where}: unknown mlp kind '{fk}' (moe)")
                rr, er = _obj(fr, "router", f"{where}: mlp"), _obj(fr, "expert", f"{where}: mlp")
                mlp = MoeSizes(experts=rr.integer("experts", minimum=1), top=rr.integer("top", minimum=1),
                               ff=er.integer("ff", minimum=1), limit=er.number("limit"))
                if mlp.top > mlp.experts:
                    raise ConfigError(f"{where}: top {mlp.top} of {mlp.experts} experts")
                if not mlp.limit > 0:
                    raise ConfigError(f"{where}: the experts' limit must be positive, got {mlp.limit}")
            out.append(LenesunLayer(kind, m, mlp))
        return LenesunConfig(
            architecture=r.string("architecture"), vocab=r.integer("vocab", minimum=1),
            width=r.integer("width", minimum=1), eps=norm.number("eps"),
            residual_mult=r.number("residual_mult"), embedding_scale=emb.number("scale"), layers=tuple(out))
