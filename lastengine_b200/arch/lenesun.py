"""The Lenesun decoder as a plan.

x = embed[token] * s.  A layer is the parallel arrangement (parts.block): h = norm(x) with a layer norm
(weight, no bias), x += m * (mixer(h) + ff(h)).  The mixer is latent attention (parts.latent_attention)
with a sink logit per head and adjacent-pair rotation of the rotated query/key part; a layer may read
the rows an earlier layer cached instead of projecting its own (its schedule entry names that layer's
cache entry and writes nothing).  The feed-forward is a mixture of experts: the k largest router
logits (bias inside the logit) weighted by the softmax over the chosen ones, experts
y = g sigmoid(1.702 g) (u + 1) with g = min(gate, limit), u = clamp(up, -limit, limit).  The model's
layer norm, then logits against the embedding table itself (not scaled).

Tensor names: embed, final.norm, and per layer l<i>.norm1, l<i>.mix.{dq, dq.norm, uq, dkv, dkv.norm,
uk, uv, sink, o}, l<i>.mlp.{router, router.b, e<j>.gate, e<j>.up, e<j>.down}.
"""
from __future__ import annotations

import re

from ..config.lenesun import LenesunConfig
from ..parts.base import LayerSpec, ModelPlan, PartSpec, ScheduleEntry
from ..registry import ARCHITECTURES

NAMES = ("Lenesun", "lenesun")

EXPERT_SIGMOID_SLOPE = 1.702      # the design's constant in g * sigmoid(1.702 g)

# names that are a part's prefix in the plan and a tensor in the checkpoint
_BARE = re.compile(r"^(embed|final\.norm|l\d+\.norm1)$")


def _alias(name: str) -> str:
    return name + ".weight" if _BARE.match(name) else name


def _checkpoint_name(canonical: str) -> str:
    return canonical[: -len(".weight")] if canonical.endswith(".weight") and _BARE.match(canonical[: -len(".weight")]) \
        else canonical


def lenesun_plan(cfg: LenesunConfig) -> ModelPlan:
    W = cfg.width
    norm = PartSpec("layernorm", {"size": W, "eps": cfg.eps})
    layers: list[LayerSpec] = []
    schedule: list[ScheduleEntry] = []
    for i, lay in enumerate(cfg.layers):
        m = lay.mixer
        position = PartSpec("rope", {"rope_dim": m.rot.dims, "theta": m.rot.base, "style": "adjacent"}) \
            if m.rot.dims else PartSpec("none")
        mixer = PartSpec("latent_attention", {
            "hidden_size": W, "num_heads": m.heads, "head_dim": m.dim, "rope_dim": m.rot_dim, "v_head_dim": m.vdim,
            "q_rank": m.q_rank, "kv_rank": m.kv_rank, "norm_eps": cfg.eps, "scale": m.scale, "position": position,
            "sink": True, "own_kv": m.kv_from is None})
        ffn = None
        if lay.mlp is not None:
            f = lay.mlp
            ffn = PartSpec("topk_moe", {
                "hidden_size": W, "num_experts": f.experts, "top_k": f.top, "expert_size": f.ff,
                "router": "softmax_chosen", "use_bias": True, "activation": "clamped_sigmoid",
                "limit": f.limit, "alpha": EXPERT_SIGMOID_SLOPE,
                "names": {"router": "router", "bias": "router.b", "gate": "e{e}.gate", "up": "e{e}.up",
                          "down": "e{e}.down"}})
        layers.append(LayerSpec(
            prefix=f"l{i}", mixer=mixer, ffn=ffn, mixer_norm=norm, ffn_norm=None, block="parallel_residual",
            block_params={"mult": cfg.residual_mult}, names={"mixer": "mix", "ffn": "mlp", "mixer_norm": "norm1"}))
        # one schedule entry per layer, so a layer's number is its cache entry's number too
        schedule.append(ScheduleEntry(i) if m.kv_from is None else ScheduleEntry(i, cache=m.kv_from, writes_cache=False))
    return ModelPlan(
        architecture=cfg.architecture, hidden_size=W, vocab_size=cfg.vocab,
        embedding=PartSpec("token_embedding", {"vocab_size": cfg.vocab, "hidden_size": W, "scale": cfg.embedding_scale}),
        final_norm=norm,
        head=PartSpec("linear_head", {"vocab_size": cfg.vocab, "hidden_size": W, "tied": True}),
        layers=layers, schedule=schedule,
        names={"embedding": "embed", "final_norm": "final.norm", "head": "head"},
        tensor_aliases=_alias, checkpoint_names=_checkpoint_name,
        init_std=0.05, init_stds={".sink": 1.0, ".router": 0.3})


@ARCHITECTURES.register(*NAMES)
def build_lenesun(raw: dict) -> ModelPlan:
    return lenesun_plan(LenesunConfig.from_dict(raw))
