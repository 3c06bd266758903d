"""The Zekivik decoder as a plan.

A layer is the gated pre-norm arrangement (parts.block): x += s1 * mixer(n1(x)) and, where the
layer has a feed-forward, x += s2 * ff(n2(x)); the norms store their weight around zero (factor
1 + w), the gates s = sigmoid(R h + b) read the sublayer's own input.  Mixers: softmax attention
with a short causal convolution on q, k and v, unit-norm q, k and v, grouped key/value heads, value
heads of their own width and a sigmoid gate per head; or retention (decayed linear attention with a
float state).  The feed-forward is gated with the tanh form of gelu.

A range of layers may run several times in a row with the same weights; every run of a layer is a
schedule entry with a cache entry of its own.  Before every pass over the range but the first, the
embedding output is added to the residual stream, and before every pass, the first too, the pass's
row of the table `loop.step` (stream additions of the plan).

Tensor names: embed, head, final.norm, loop.step, and per layer l<i>.norm1/.norm2, l<i>.rg1(.b),
l<i>.rg2(.b), l<i>.mix.{q,k,v,g,o} with l<i>.mix.{q,k,v}.conv for attention, l<i>.mlp.{gate,up,down}.
"""
from __future__ import annotations

import re

from ..config.zekivik import ATTENTION, ZekivikConfig
from ..parts.base import LayerSpec, ModelPlan, PartSpec, ScheduleEntry, StreamAdd
from ..registry import ARCHITECTURES

NAMES = ("Zekivik", "zekivik")
LOOP_TABLE = "loop.step"

# names that are a part's prefix in the plan and a tensor in the checkpoint
_BARE = re.compile(r"^(embed|head|final\.norm|l\d+\.norm[12])$")


def _alias(name: str) -> str:
    return name + ".weight" if _BARE.match(name) else name


def _checkpoint_name(canonical: str) -> str:
    return canonical[: -len(".weight")] if canonical.endswith(".weight") and _BARE.match(canonical[: -len(".weight")]) \
        else canonical


def zekivik_plan(cfg: ZekivikConfig) -> ModelPlan:
    W = cfg.width
    norm = PartSpec("rmsnorm", {"size": W, "eps": cfg.eps, "offset": 1.0})
    gate = lambda: PartSpec("sigmoid_gate", {"hidden_size": W, "tensor": "", "bias_tensor": "b"})  # noqa: E731
    layers: list[LayerSpec] = []
    for i, lay in enumerate(cfg.layers):
        m = lay.mixer
        position = PartSpec("rope", {"rope_dim": m.rot.dims, "theta": m.rot.base, "style": "neox"}) \
            if m.rot.dims else PartSpec("none")
        if lay.type == ATTENTION:
            mixer = PartSpec("attention", {
                "hidden_size": W, "num_heads": m.heads, "num_kv_heads": m.kv_heads, "head_dim": m.dim,
                "v_head_dim": m.vdim, "norm_eps": cfg.eps, "qk_norm": "unit", "v_norm": True,
                "conv_taps": m.conv, "scale": m.scale, "output_gate": True, "position": position,
                "names": {"q": "q", "k": "k", "v": "v", "o": "o", "gate": "g",
                          "q_conv": "q.conv", "k_conv": "k.conv", "v_conv": "v.conv"}})
        else:
            mixer = PartSpec("retention", {
                "hidden_size": W, "num_heads": m.heads, "head_dim": m.dim, "v_head_dim": m.vdim,
                "decay": list(m.decay), "norm_eps": cfg.eps, "position": position,
                "names": ("q", "k", "v", "g", "o")})
        ffn = None if lay.ff is None else PartSpec("gated_dense", {
            "hidden_size": W, "intermediate_size": lay.ff, "activation": "gelu_tanh", "names": ("gate", "up", "down")})
        gates = {"mixer_gate": gate()}
        if ffn is not None:
            gates["ffn_gate"] = gate()
        layers.append(LayerSpec(
            prefix=f"l{i}", mixer=mixer, ffn=ffn, mixer_norm=norm, ffn_norm=None if ffn is None else norm,
            block="gated_pre_norm_residual", gates=gates,
            names={"mixer": "mix", "ffn": "mlp", "mixer_norm": "norm1", "ffn_norm": "norm2",
                   "mixer_gate": "rg1", "ffn_gate": "rg2"}))
    schedule, adds = [], []
    for at, (layer, opens) in enumerate(cfg.runs()):
        schedule.append(ScheduleEntry(layer))
        if opens is not None:
            adds.append(StreamAdd(before=at, embedding=opens > 0, table=LOOP_TABLE, row=opens))
    tables = {LOOP_TABLE: (cfg.loop.times, W)} if adds else {}
    return ModelPlan(
        architecture=cfg.architecture, hidden_size=W, vocab_size=cfg.vocab,
        embedding=PartSpec("token_embedding", {"vocab_size": cfg.vocab, "hidden_size": W}),
        final_norm=norm,
        head=PartSpec("linear_head", {"vocab_size": cfg.vocab, "hidden_size": W, "tied": False}),
        layers=layers, schedule=schedule,
        names={"embedding": "embed", "final_norm": "final.norm", "head": "head"},
        tensor_aliases=_alias, checkpoint_names=_checkpoint_name,
        stream_adds=tuple(adds), stream_tables=tables,
        unused_tensors=() if adds else (LOOP_TABLE,),      # a checkpoint may carry the table of a loop over no layers
        # the model keeps its signal through the looped passes with weights of this size
        init_std=0.05, init_stds={".conv": 0.5, LOOP_TABLE: 0.3})


@ARCHITECTURES.register(*NAMES)
def build_zekivik(raw: dict) -> ModelPlan:
    return zekivik_plan(ZekivikConfig.from_dict(raw))
