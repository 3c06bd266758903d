"""Grouped-query attention mixer over the paged cache.

q = Wq h, k = Wk h, v = Wv h; optional per-head RMSNorm on q and k (shared [head_dim] weights,
the model's eps) before the rotation; k and v appended to the cache at the token's position;
causal softmax attention with scale 1/sqrt(head_dim), optionally inside a window; optional
sigmoid gate per head from its own projection; out = Wo o.  (src/dense.rs:113-152.)
The three projections (and the gate) are one matrix product over fused weights, as the
reference fuses gate and up (src/gpu/dense.rs:67-74).

Options other designs use: value heads of a width of their own (`v_head_dim`); a short causal
depthwise convolution over time on every channel of q, k and v right after the projection
(`conv_taps` > 1; taps `<tensor>.conv` [channels, taps]; the last taps-1 projected values of a
sequence are state beside its keys and values); q and k divided by their root mean square without
a weight (`qk_norm="unit"`); every value head divided by its root mean square before it is cached
(`v_norm`).  The kernels norm before they rotate; a design that rotates first gets the same
numbers, since a rotation of pairs leaves the head's sum of squares as it was.  `names` renames
the tensors under the part's prefix.

Key and value heads of different widths are cached at the wider of the two when that is a size the
tensor-core attention kernels take: the narrower heads are stored with zeros behind them (a zero
dimension changes no score and adds nothing to a value; the scale is explicit and the norms run over
the head as it is), and the output projection gets zero columns where the padding is.  Other pairs
of widths run the general kernel.
"""
from __future__ import annotations

import math

import torch

from ..ops import kernels
from ..registry import MIXERS, POSITION_ENCODINGS
from .base import MATRIX, NORM, VECTOR, BuildEnv, KVSpec, Mixer, PartSpec, StateSpec, TensorSpec


@MIXERS.register("attention")
class AttentionMixer(Mixer):
    split_norm = True

    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int,
                 norm_eps: float, qk_norm: bool = True, position: PartSpec | None = None,
                 window: int = 0, output_gate: bool = False, own_kv: bool = True,
                 scale: float | None = None, v_head_dim: int | None = None, conv_taps: int = 0,
                 v_norm: bool = False, names: dict[str, str] | None = None):
        if num_heads % num_kv_heads != 0:
            raise ValueError(f"{num_heads} heads do not divide into {num_kv_heads} kv heads")
        if head_dim > 256:
            raise ValueError(f"head_dim {head_dim} is larger than the attention kernels take (256)")
        self.D, self.nh, self.nkv, self.hd = int(hidden_size), int(num_heads), int(num_kv_heads), int(head_dim)
        self.eps = float(norm_eps)
        self.qk_unit = qk_norm == "unit"            # divided by the root mean square, no weight
        self.qk_norm = bool(qk_norm) and not self.qk_unit
        self.vd = self.hd if v_head_dim is None else int(v_head_dim)
        if self.vd > 256:
            raise ValueError(f"v_head_dim {self.vd} is larger than the attention kernels take (256)")
        # widths in the cache: the wider of the two where the fast kernels take it
        wide = max(self.hd, self.vd)
        self.khd, self.kvd = (wide, wide) if self.hd != self.vd and wide in (32, 64, 96, 128) else (self.hd, self.vd)
        self.taps = int(conv_taps)
        if not 0 <= self.taps <= 16:
            raise ValueError(f"conv_taps {conv_taps}: 0 (no convolution) or 1..16")
        if self.taps and not own_kv:
            raise ValueError("a layer that reads another layer's cache cannot convolve its own k and v")
        self.v_norm = bool(v_norm)
        self.n = {"q": "q_proj.weight", "k": "k_proj.weight", "v": "v_proj.weight", "o": "out_proj.weight",
                  "gate": "gate_proj.weight", "q_norm": "q_layernorm.weight", "k_norm": "k_layernorm.weight",
                  "q_conv": "q_conv.weight", "k_conv": "k_conv.weight", "v_conv": "v_conv.weight"}
        self.n.update(names or {})
        self.window = int(window)
        self.output_gate = bool(output_gate)
        self.own_kv = bool(own_kv)
        self.scale = float(scale) if scale is not None else 1.0 / math.sqrt(self.hd)
        pos = position or PartSpec("none")
        self.position = POSITION_ENCODINGS.get(pos.kind)(**pos.params)
        self.w_in = self.w_out = self.q_norm_w = self.k_norm_w = None
        self.n_extra, self.extra_out = 0, None

    def tensors(self) -> dict[str, TensorSpec]:
        D, nh, nkv, hd, vd, n = self.D, self.nh, self.nkv, self.hd, self.vd, self.n
        t = {n["q"]: TensorSpec((nh * hd, D), MATRIX),
             n["o"]: TensorSpec((D, nh * vd), MATRIX)}
        if self.own_kv:
            t[n["k"]] = TensorSpec((nkv * hd, D), MATRIX)
            t[n["v"]] = TensorSpec((nkv * vd, D), MATRIX)
        if self.qk_norm:
            t[n["q_norm"]] = TensorSpec((hd,), NORM)
            if self.own_kv:
                t[n["k_norm"]] = TensorSpec((hd,), NORM)
        if self.output_gate:
            t[n["gate"]] = TensorSpec((nh, D), MATRIX)
        if self.taps:
            t[n["q_conv"]] = TensorSpec((nh * hd, self.taps), VECTOR, std=0.5)
            t[n["k_conv"]] = TensorSpec((nkv * hd, self.taps), VECTOR, std=0.5)
            t[n["v_conv"]] = TensorSpec((nkv * vd, self.taps), VECTOR, std=0.5)
        for name, spec in self.position.tensors().items():
            t[f"position.{name}"] = spec
        return t

    def cache_spec(self):
        kv = KVSpec(self.nkv, self.khd, self.window, None if self.kvd == self.khd else self.kvd)
        if self.taps <= 1:       # a single tap looks at the current row only
            return kv
        # the convolution's memory: the last taps-1 projected values of every q, k and v channel
        return kv, StateSpec(((self.nh + self.nkv) * self.hd + self.nkv * self.vd, self.taps - 1), torch.float32)

    def load(self, tensors, env: BuildEnv) -> None:
        n = self.n
        parts = [tensors[n["q"]]]
        if self.own_kv:
            parts += [tensors[n["k"]], tensors[n["v"]]]
        if self.output_gate:
            parts.append(tensors[n["gate"]])
        self.w_in = torch.cat(parts, dim=0).contiguous() if len(parts) > 1 else parts[0].contiguous()
        self.w_out = tensors[n["o"]].contiguous()
        if self.kvd != self.vd:      # zero columns where the cached value heads are wider than the heads
            w = torch.zeros((self.D, self.nh, self.kvd), dtype=self.w_out.dtype, device=self.w_out.device)
            w[:, :, : self.vd] = self.w_out.view(self.D, self.nh, self.vd)
            self.w_out = w.view(self.D, self.nh * self.kvd).contiguous()
        if self.qk_norm:
            self.q_norm_w = tensors[n["q_norm"]].contiguous()
            self.k_norm_w = tensors[n["k_norm"]].contiguous() if self.own_kv else None
        elif self.qk_unit:
            self.q_norm_w = self.k_norm_w = torch.ones(self.hd, dtype=torch.float32, device=env.device)
        self.w_conv = None
        if self.taps:
            self.w_conv = torch.cat([tensors[n["q_conv"]], tensors[n["k_conv"]], tensors[n["v_conv"]]],
                                    dim=0).to(torch.float32).contiguous()
        self.position.load({n[len("position."):]: v for n, v in tensors.items() if n.startswith("position.")}, env)

    def split_reader_weight(self):
        return self.w_in

    def absorb_input_rows(self, w: torch.Tensor) -> bool:
        """Takes the rows of another product over the same input (a gate on this mixer's result) into
        the fused projection; every forward then leaves their result in `extra_out` [rows, len(w)]."""
        if not self.own_kv or w.dtype != self.w_in.dtype or w.shape[1] != self.D or self.n_extra:
            return False
        self.w_in = torch.cat([self.w_in, w], dim=0).contiguous()
        self.n_extra = int(w.shape[0])
        return True

    def flops_per_query_key(self) -> int:
        return 2 * self.nh * (self.khd + self.kvd)    # a score and a weighted value, a multiply-add each, per head and dimension

    def forward(self, h, out, accumulate, batch, cache, env) -> None:
        nh, nkv, hd, vd = self.nh, self.nkv, self.hd, self.vd
        plain_v = vd == hd and not self.v_norm
        M = h.shape[0]
        ws = env.workspace
        scale, emit = env.take_split_in(), env.take_split_out()
        writes = self.own_kv and cache.writable
        if self.own_kv and not cache.writable:
            w_in = self.w_in[: nh * hd] if not (self.output_gate or self.n_extra) else None
        else:
            w_in = self.w_in
        if w_in is None:  # q and gate rows are not adjacent once k, v are skipped: two products
            raise NotImplementedError("a gated attention layer reading another layer's cache")
        proj = ws.get("attn.proj", (M, w_in.shape[0]), env.dtype)
        kernels.linear(proj, h, w_in, scale=scale)
        q_in = proj[:, : nh * hd]
        k_in = v_in = gate = None
        col = nh * hd
        if writes:
            k_in = proj[:, col: col + nkv * hd]
            v_in = proj[:, col + nkv * hd: col + nkv * (hd + vd)]
            col += nkv * (hd + vd)
        if self.output_gate:
            gate = proj[:, col: col + nh]
        if self.n_extra:
            self.extra_out = proj[:, proj.shape[1] - self.n_extra:]
        if self.taps:
            # q, k and v (not the gate) through the short convolution; the state moves on by the step's rows
            if not writes:
                raise NotImplementedError("a convolved attention layer that does not write its cache")
            conv = ws.get("attn.conv", (M, col), env.dtype)
            kernels.causal_conv(conv, proj[:, :col], self.w_conv, cache.state, batch)
            q_in, k_in = conv[:, : nh * hd], conv[:, nh * hd: (nh + nkv) * hd]
            v_in = conv[:, (nh + nkv) * hd:]
        khd, kvd = self.khd, self.kvd
        q = ws.get("attn.q", (M, nh * khd), env.dtype)
        kp, vp = (cache.k, cache.v) if writes else (None, None)
        rotary = self.position.fused_rotary()
        raw = None
        if (rotary is not None and plain_v and khd == hd
                and kernels.decode_attention_takes_raw(env.dtype, batch, M, nh, nkv, hd, cache.page_size, *rotary)):
            # a decode step: the attention kernel norms and rotates q and k and stores k and v itself
            raw = kernels.RawQKV(q_in, k_in, v_in, self.q_norm_w, self.k_norm_w if writes else None, self.eps, *rotary)
        elif rotary is not None:
            # per-head norm, rotation and the cache write in one launch
            kernels.qk_rope_store(q, q_in, k_in, v_in, kp, vp, cache.block_table, batch, self.q_norm_w,
                                  self.k_norm_w if writes else None, self.eps, *rotary, nh, nkv, khd, cache.page_size,
                                  vd=kvd, v_norm=self.v_norm, hd_in=hd, vd_in=vd)
        elif not plain_v:
            raise NotImplementedError("value heads of their own width or norm with a position encoding that is no rotation")
        else:
            # an encoding of the part's own: norm, then the part on the normed q and k, then the store
            qn = ws.get("attn.qn", (M, nh * hd), env.dtype)
            kernels.qk_rope_store(qn, q_in, None, None, None, None, cache.block_table, batch, self.q_norm_w, None,
                                  self.eps, None, 0, True, nh, nkv, hd, cache.page_size)
            kn = vn = None
            if writes:
                kn = ws.get("attn.kn", (M, nkv * hd), env.dtype)
                kernels.qk_rope_store(kn, k_in, None, None, None, None, cache.block_table, batch, self.k_norm_w, None,
                                      self.eps, None, 0, True, nkv, nkv, hd, cache.page_size)
                vn = ws.get("attn.vn", (M, nkv * hd), env.dtype)      # the values beside them, rows as wide as kn's
                kernels.qk_rope_store(vn, v_in, None, None, None, None, cache.block_table, batch, None, None,
                                      self.eps, None, 0, True, nkv, nkv, hd, cache.page_size)
            self.position.apply(qn.view(M, nh, hd), kn.view(M, nkv, hd) if writes else None, batch.row_pos)
            kernels.qk_rope_store(q, qn, kn, vn, kp, vp, cache.block_table, batch, None, None, self.eps,
                                  None, 0, True, nh, nkv, hd, cache.page_size)
        o = ws.get("attn.o", (M, nh * kvd), env.dtype)
        n_splits = kernels.attention_splits(batch, nkv, nh // nkv, hd=khd)
        scratch = None
        if n_splits > 1:
            scratch = ws.get("attn.part", (M * nh * n_splits * (max(khd, kvd) + 2),), torch.float32)
        kernels.attention(o, None if raw is not None else q, cache.k, cache.v, cache.block_table, batch, nh, nkv, khd,
                          cache.page_size, self.window, self.scale, gate=gate, n_splits=n_splits, scratch=scratch, raw=raw,
                          vd=kvd)
        kernels.linear(out, o, self.w_out, kernels.ACCUMULATE if accumulate else kernels.STORE,
                       emit=emit if accumulate else None)
