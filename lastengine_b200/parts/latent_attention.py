"""Latent attention: queries, keys and values go through low-rank latents, and only the key/value
latent is cached.

    c_q = rmsnorm(W_dq h) * g_q                 [q_rank]
    q_h = W_uq,h c_q = [q_h^n | q_h^r]          per head: `head_dim` unrotated, `rope_dim` rotated numbers
    [a | r] = W_dkv h;  c = rmsnorm(a) * g_kv   [rank];  k^r = rotate(r)  [rope_dim], one for all heads
    k_h = W_uk,h c,  v_h = W_uv,h c             per head: `head_dim` and `v_head_dim` numbers
    s_h(i, j) = scale * (q_h^n(i) . k_h(j) + q_h^r(i) . k^r(j)),  j <= i
    p = softmax over the row's scores and, with `sink`, one learned logit per head that has neither key
        nor value (it only takes its share of the denominator)
    out = W_o [sum_j p_h(i, j) v_h(j)]_h

The rotation pairs dimension 2i with 2i + 1 over the first `rot_dims` of the rotated part (the
position encoding part, adjacent style, says which and by what angles); q^r and r are rotated, v is not.

What is cached per position is the row [c | k^r] (`LatentSpec`), however many heads there are.  A
layer with `own_kv=False` has no W_dkv: it reads the rows another layer cached, with its own W_uk and
W_uv (the plan names that layer's cache entry in the schedule).

The kernels never form k_h or v_h.  q_h^n . (W_uk,h c) = (W_uk,h^T q_h^n) . c, so each query is taken
into the latent space by a product grouped by head, attention runs with the cached row as every
head's key and its first `rank` numbers as every head's value, and the per-head results go through
W_uv,h in a second grouped product before the output projection.  A step therefore reads each cached
row once for all heads, and a prompt and a decode step run the same kernels.
"""
from __future__ import annotations

import torch

from ..ops import kernels
from ..registry import MIXERS, POSITION_ENCODINGS
from .base import MATRIX, NORM, VECTOR, BuildEnv, LatentSpec, Mixer, PartSpec, TensorSpec


_HEAD_OFFSETS: dict[tuple, torch.Tensor] = {}


def _up8(n: int) -> int:
    return -(-n // 8) * 8


@MIXERS.register("latent_attention")
class LatentAttentionMixer(Mixer):
    def __init__(self, hidden_size: int, num_heads: int, head_dim: int, rope_dim: int, v_head_dim: int,
                 q_rank: int, kv_rank: int, norm_eps: float, scale: float, position: PartSpec | None = None,
                 sink: bool = False, own_kv: bool = True, names: dict[str, str] | None = None):
        self.D, self.H = int(hidden_size), int(num_heads)
        self.hd, self.rd, self.vd = int(head_dim), int(rope_dim), int(v_head_dim)
        self.q_rank, self.rank = int(q_rank), int(kv_rank)
        if min(self.H, self.hd, self.vd, self.q_rank, self.rank) < 1 or self.rd < 0:
            raise ValueError("latent attention: every size must be positive (rope_dim may be 0)")
        if self.rank > 512 or self.rd > 256:
            raise ValueError(f"latent attention: kv_rank {self.rank} / rope_dim {self.rd} beyond what the kernel takes (512 / 256)")
        self.eps, self.scale = float(norm_eps), float(scale)
        self.has_sink, self.own_kv = bool(sink), bool(own_kv)
        self.n = {"dq": "dq", "dq_norm": "dq.norm", "uq": "uq", "dkv": "dkv", "dkv_norm": "dkv.norm",
                  "uk": "uk", "uv": "uv", "o": "o", "sink": "sink"}
        self.n.update(names or {})
        pos = position or PartSpec("none")
        self.position = POSITION_ENCODINGS.get(pos.kind)(**pos.params)
        self.w_down = self.w_uq = self.w_ukt = self.w_uv = self.w_o = None
        self.q_norm_w = self.kv_norm_w = self.sink = None
        self.inv_freq, self.rot_dims = None, 0

    def tensors(self) -> dict[str, TensorSpec]:
        n, H = self.n, self.H
        t = {n["dq"]: TensorSpec((self.q_rank, self.D), MATRIX),
             n["dq_norm"]: TensorSpec((self.q_rank,), NORM),
             n["uq"]: TensorSpec((H * (self.hd + self.rd), self.q_rank), MATRIX),
             n["uk"]: TensorSpec((H * self.hd, self.rank), MATRIX),
             n["uv"]: TensorSpec((H * self.vd, self.rank), MATRIX),
             n["o"]: TensorSpec((self.D, H * self.vd), MATRIX)}
        if self.own_kv:
            t[n["dkv"]] = TensorSpec((self.rank + self.rd, self.D), MATRIX)
            t[n["dkv_norm"]] = TensorSpec((self.rank,), NORM)
        if self.has_sink:
            t[n["sink"]] = TensorSpec((H,), VECTOR)
        for name, spec in self.position.tensors().items():
            t[f"position.{name}"] = spec
        return t

    def cache_spec(self):
        return LatentSpec(self.rank, self.rd)

    def load(self, tensors, env: BuildEnv) -> None:
        n, H = self.n, self.H
        # the down projections are one product: [W_dq ; W_dkv]
        self.w_down = (torch.cat([tensors[n["dq"]], tensors[n["dkv"]]], dim=0) if self.own_kv else tensors[n["dq"]]).contiguous()
        self.w_uq = tensors[n["uq"]].contiguous()
        # per head, W_uk^T [rank, head_dim] (the product that takes a query into the latent space) and
        # W_uv [v_head_dim, rank]; inner sizes filled up with zeros to what the grouped products fetch at a time
        self.hd_p = self.hd if env.is_float32 else _up8(self.hd)
        self.rank_p = self.rank if env.is_float32 else _up8(self.rank)
        uk = tensors[n["uk"]].view(H, self.hd, self.rank)
        self.w_ukt = torch.zeros((H, self.rank, self.hd_p), dtype=uk.dtype, device=uk.device)
        self.w_ukt[:, :, : self.hd] = uk.transpose(1, 2)
        uv = tensors[n["uv"]].view(H, self.vd, self.rank)
        self.w_uv = torch.zeros((H, self.vd, self.rank_p), dtype=uv.dtype, device=uv.device)
        self.w_uv[:, :, : self.rank] = uv
        self.w_o = tensors[n["o"]].contiguous()
        self.q_norm_w = tensors[n["dq_norm"]].to(torch.float32).contiguous()
        self.kv_norm_w = tensors[n["dkv_norm"]].to(torch.float32).contiguous() if self.own_kv else None
        self.sink = tensors[n["sink"]].to(torch.float32).contiguous() if self.has_sink else None
        self.position.load({k[len("position."):]: v for k, v in tensors.items() if k.startswith("position.")}, env)
        rotary = self.position.fused_rotary()
        if rotary is None:
            raise NotImplementedError("latent attention with a position encoding that is no rotation")
        inv_freq, rot_dims, neox = rotary
        if inv_freq is not None:
            if neox:
                raise NotImplementedError("latent attention rotates adjacent pairs; the encoding asks for split halves")
            if rot_dims > self.rd:
                raise ValueError(f"{rot_dims} rotated dimensions in a rotated part of {self.rd}")
            self.inv_freq, self.rot_dims = inv_freq, int(rot_dims)

    def flops_per_row(self) -> int:
        H = self.H
        # W_uk is applied once per row (to the query) and W_uv once (to the result), not once per cached position
        n = self.q_rank * self.D + H * (self.hd + self.rd) * self.q_rank + H * self.hd * self.rank \
            + H * self.vd * self.rank + self.D * H * self.vd
        if self.own_kv:
            n += (self.rank + self.rd) * self.D
        return 2 * n

    def flops_per_query_key(self) -> int:
        return 2 * self.H * (2 * self.rank + self.rd)   # a score over the cached row and a weighted sum of its latent

    def _head_offsets(self, M: int, device) -> torch.Tensor:
        """Row ranges of the head-major buffers for the grouped products: head h owns rows [h M, (h + 1) M).
        Made once per (heads, rows) and kept for good (a few bytes each): captured steps hold their addresses."""
        key = (self.H, M, str(device))
        t = _HEAD_OFFSETS.get(key)
        if t is None:
            t = _HEAD_OFFSETS[key] = (torch.arange(self.H + 1, dtype=torch.int64) * M).to(torch.int32).to(device)
        return t

    def forward(self, h, out, accumulate, batch, cache, env) -> None:
        H, hd, rd, vd, rank = self.H, self.hd, self.rd, self.vd, self.rank
        M = h.shape[0]
        ws = env.workspace
        writes = self.own_kv and cache.writable
        if self.own_kv and not cache.writable:
            raise NotImplementedError("a latent-attention layer with its own W_dkv scheduled to read another entry's cache")
        pool = cache.k[:, 0]                       # [page, page_size, rank + rope_dim]
        if pool.shape[-1] != rank + rd:
            raise ValueError(f"the cache rows are {pool.shape[-1]} wide, this layer reads {rank} + {rd}")
        proj = ws.get("lat.proj", (M, self.w_down.shape[0]), env.dtype)
        kernels.linear(proj, h, self.w_down)
        cq = ws.get("lat.cq", (M, self.q_rank), env.dtype)
        kernels.latent_prep(cq, proj, pool if writes else None, cache.block_table, batch, self.q_norm_w,
                            self.kv_norm_w, self.eps, self.inv_freq, self.rot_dims, rank, rd, cache.page_size)
        q = ws.get("lat.q", (M, H * (hd + rd)), env.dtype)
        kernels.linear(q, cq, self.w_uq)
        qn = ws.get("lat.qn", (H, M, self.hd_p), env.dtype)
        qr = ws.get("lat.qr", (M, H, rd), env.dtype)
        kernels.latent_q_split(qn, qr, q, batch.row_pos, self.inv_freq, self.rot_dims, H, hd, rd)
        offsets = self._head_offsets(M, h.device)
        qt = ws.get("lat.qt", (H, M, rank), env.dtype)
        kernels.linear(qt.view(H * M, rank), qn.view(H * M, self.hd_p), self.w_ukt, group_offsets=offsets, rows_hint=H * M)
        u = ws.get("lat.u", (H, M, self.rank_p), env.dtype)
        mma = kernels.latent_attention_uses_mma(env.dtype, rank, rd, cache.page_size, self.rank_p)
        n_splits = kernels.latent_attention_splits(batch, H, mma, rank)
        scratch = ws.get("lat.part", (M * H * n_splits * (rank + 2),), torch.float32) if n_splits > 1 else None
        kernels.latent_attention(u, qt, qr, pool, cache.block_table, batch, self.sink, rank, rd, cache.page_size,
                                 self.scale, n_splits=n_splits, scratch=scratch)
        v = ws.get("lat.v", (H, M, vd), env.dtype)
        kernels.linear(v.view(H * M, vd), u.view(H * M, self.rank_p), self.w_uv, group_offsets=offsets, rows_hint=H * M)
        if M == 1:
            o = v.view(1, H * vd)                  # one row: head-major and row-major are the same memory
        else:
            o = ws.get("lat.o", (M, H * vd), env.dtype)
            kernels.heads_to_rows(o, v)
        kernels.linear(out, o, self.w_o, kernels.ACCUMULATE if accumulate else kernels.STORE)
