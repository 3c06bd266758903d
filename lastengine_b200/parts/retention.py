"""Retention mixer: linear attention with a fixed decay per head, without softmax or denominator.

q = Wq h, k = Wk h (heads x dim), v = Wv h, g = Wg h (heads x vdim), one product over the fused
weights.  q and k are rotated by position (the position encoding's table, on its first rope_dim
dimensions of each head), k is scaled by `k_scale` (dim^-1/2 unless given); per head
    S_t = decay_h S_{t-1} + k_t v_t^T,    o_t = S_t^T q_t,
each head's o_t is divided by its root mean square (eps, no weight), the heads side by side are
multiplied by silu(g) and projected by Wo.  The state S [heads, dim, vdim] is float, zero at a
sequence's start and carried per cache slot; everything between the projections is float.
A prompt runs the chunked kernels (ops.kernels.retention chooses), a decode step the recurrent one.
"""
from __future__ import annotations

import torch

from ..ops import kernels
from ..registry import MIXERS, POSITION_ENCODINGS
from .base import MATRIX, BuildEnv, Mixer, PartSpec, StateSpec, TensorSpec


@MIXERS.register("retention")
class RetentionMixer(Mixer):
    def __init__(self, hidden_size: int, num_heads: int, head_dim: int, v_head_dim: int, decay: list[float],
                 norm_eps: float, position: PartSpec | None = None, k_scale: float | None = None,
                 names: tuple[str, str, str, str, str] = ("q_proj.weight", "k_proj.weight", "v_proj.weight",
                                                          "g_proj.weight", "out_proj.weight")):
        self.D, self.H, self.d, self.e = int(hidden_size), int(num_heads), int(head_dim), int(v_head_dim)
        if len(decay) != self.H:
            raise ValueError(f"{len(decay)} decay constants for {self.H} heads")
        if not all(0.0 <= float(x) <= 1.0 for x in decay):
            raise ValueError(f"decay constants outside [0, 1]: {decay}")
        if self.d > 1024 or self.e > 1024:
            raise ValueError(f"head sizes {self.d} x {self.e} are larger than the retention kernels take (1024)")
        self.decay_values = [float(x) for x in decay]
        self.eps = float(norm_eps)
        self.k_scale = float(k_scale) if k_scale is not None else self.d ** -0.5
        pos = position or PartSpec("none")
        self.position = POSITION_ENCODINGS.get(pos.kind)(**pos.params)
        self.names = tuple(str(n) for n in names)
        self.w_in = self.w_out = self.decay = None
        self.n_extra, self.extra_out = 0, None

    def tensors(self) -> dict[str, TensorSpec]:
        D, H, d, e = self.D, self.H, self.d, self.e
        nq, nk, nv, ng, no = self.names
        t = {nq: TensorSpec((H * d, D), MATRIX), nk: TensorSpec((H * d, D), MATRIX),
             nv: TensorSpec((H * e, D), MATRIX), ng: TensorSpec((H * e, D), MATRIX),
             no: TensorSpec((D, H * e), MATRIX)}
        for name, spec in self.position.tensors().items():
            t[f"position.{name}"] = spec
        return t

    def cache_spec(self):
        return StateSpec((self.H, self.d, self.e), torch.float32)

    def load(self, tensors, env: BuildEnv) -> None:
        nq, nk, nv, ng, no = self.names
        self.w_in = torch.cat([tensors[nq], tensors[nk], tensors[nv], tensors[ng]], dim=0).contiguous()
        self.w_out = tensors[no].contiguous()
        self.decay = torch.tensor(self.decay_values, dtype=torch.float32, device=env.device)
        self.position.load({n[len("position."):]: v for n, v in tensors.items() if n.startswith("position.")}, env)
        rotary = self.position.fused_rotary()
        if rotary is None or not rotary[2]:
            raise ValueError("the retention mixer takes a split-half rotation (or none) as its position encoding")
        self.inv_freq, self.rot = rotary[0], (int(rotary[1]) if rotary[0] is not None else 0)
        if self.rot > self.d:
            raise ValueError(f"{self.rot} rotated dimensions do not fit a head of {self.d}")

    def absorb_input_rows(self, w: torch.Tensor) -> bool:
        """Takes the rows of another product over the same input (a gate on this mixer's result) into
        the fused projection; every forward then leaves their result in `extra_out` [rows, len(w)]."""
        if w.dtype != self.w_in.dtype or w.shape[1] != self.D or self.n_extra:
            return False
        self.w_in = torch.cat([self.w_in, w], dim=0).contiguous()
        self.n_extra = int(w.shape[0])
        return True

    def flops_per_row(self) -> int:
        # the projections, and per head the state's update and its product with q
        return super().flops_per_row() + 4 * self.H * self.d * self.e

    def forward(self, h, out, accumulate, batch, cache, env) -> None:
        H, d, e = self.H, self.d, self.e
        M = h.shape[0]
        ws = env.workspace
        proj = ws.get("ret.proj", (M, self.w_in.shape[0]), env.dtype)
        kernels.linear(proj, h, self.w_in)
        q, k = proj[:, : H * d], proj[:, H * d: 2 * H * d]
        v, g = proj[:, 2 * H * d: 2 * H * d + H * e], proj[:, 2 * H * d + H * e: 2 * H * (d + e)]
        if self.n_extra:
            self.extra_out = proj[:, 2 * H * (d + e):]
        o = ws.get("ret.o", (M, H * e), env.dtype)
        kernels.retention(o, q, k, v, g, cache.state, self.decay, self.inv_freq, self.rot, self.k_scale, self.eps,
                          batch, H, d, e)
        kernels.linear(out, o, self.w_out, kernels.ACCUMULATE if accumulate else kernels.STORE)
