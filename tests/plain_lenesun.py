"""A plain, slow implementation of the Lenesun decoder, for tests only.

Whole sequences, no cache, no batching, one function per mechanism, ordinary tensor arithmetic
(double precision unless told otherwise).  It shares no code with the library, and it forms every
head's keys and values from the latent explicitly, which the library never does.

The design in this file's notation.  x = E[token] * s.  A layer: h = LN(x), x += m * (A(h) + F(h)),
with LN(x) = (x - mean) / sqrt(var + eps) * w.  A is latent attention:
    cq = RMS(Dq h) * wq;  per head [qn | qr] = Uq cq;  [a | r] = Dkv h;  c = RMS(a) * wkv;  kr = R(r)
    k_h = Uk_h c,  v_h = Uv_h c,  score_h(i, j) = scale * (qn_h(i) . k_h(j) + R(qr_h(i)) . kr(j)),  j <= i
    p_h(i, .) = exp(score) / (sum_j exp(score) + exp(sink_h));  A = O [sum_j p_h(i, j) v_h(j)]_h
R turns the pairs (2t, 2t + 1), t < dims/2, by the angle pos * base^(-2t/dims).  A layer may take c and kr
from an earlier layer.  F is a mixture of experts: z = Wr h + b, the `top` largest z chosen, weights
softmax over the chosen z; expert: g = min(G h, L), u = clamp(U h, -L, L), D (g * sigmoid(1.702 g) * (u + 1)).
Logits = E LN_final(x).

`rnd` is a rounding hook: the identity for the 32-bit path, rounding to bfloat16 where a bfloat16
computation stores a value.
"""
from __future__ import annotations

import json
import math
import struct

import numpy as np
import torch


def read_safetensors(path: str, dtype=torch.float64) -> dict[str, torch.Tensor]:
    with open(path, "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(n))
        data = f.read()
    out = {}
    for name, e in header.items():
        if name == "__metadata__":
            continue
        b, t = e["data_offsets"]
        if e["dtype"] == "BF16":
            arr = np.frombuffer(data[b:t], dtype=np.uint16).reshape(e["shape"])
            ten = torch.from_numpy((arr.astype(np.uint32) << 16).view(np.float32).copy())
        elif e["dtype"] == "F32":
            ten = torch.from_numpy(np.frombuffer(data[b:t], dtype=np.float32).reshape(e["shape"]).copy())
        else:
            raise ValueError(f"{name}: dtype {e['dtype']}")
        out[name] = ten.to(dtype)
    return out


def identity(t):
    return t


def round_bf16(t):
    return t.to(torch.float32).to(torch.bfloat16).to(t.dtype)


def layer_norm(x, w, eps):
    mu = x.mean(-1, keepdim=True)
    var = ((x - mu) ** 2).mean(-1, keepdim=True)
    return (x - mu) / torch.sqrt(var + eps) * w


def rms_norm(x, w, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * w


def rotate_pairs(u, pos, dims, base):
    """u [T, ..., d]: neighbouring pairs of the first `dims` numbers turned by pos * base^(-2t/dims)."""
    if dims == 0:
        return u
    out = u.clone()
    for t in range(dims // 2):
        # the design forms positions and angles in 32-bit: one rounding of the frequency, one of the product
        a = (pos.to(torch.float32) * torch.tensor(base ** (-2.0 * t / dims), dtype=torch.float32)).to(u.dtype)
        c, s = torch.cos(a), torch.sin(a)
        while c.dim() < u.dim() - 1:
            c, s = c.unsqueeze(-1), s.unsqueeze(-1)
        x, y = u[..., 2 * t], u[..., 2 * t + 1]
        out[..., 2 * t] = x * c - y * s
        out[..., 2 * t + 1] = y * c + x * s
    return out


def latent_rows(h, p, m, eps, rnd=identity):
    """What a layer caches: c [T, kv_rank] and the rotated shared key part [T, rot_dim]."""
    T = h.shape[0]
    kr_ = m["kv_rank"]
    d = rnd(h @ p["dkv"].T)
    c = rnd(rms_norm(d[:, :kr_], p["dkv.norm"], eps))
    kr = rnd(rotate_pairs(d[:, kr_:], torch.arange(T), m["rot"]["dims"], m["rot"]["base"]))
    return c, kr


def sink_softmax(s, sink):
    """s [T, T] masked scores of one head (-inf above the diagonal); the sink takes part in the denominator only."""
    mx = torch.maximum(s.max(-1, keepdim=True).values, torch.as_tensor(sink, dtype=s.dtype)) if sink is not None \
        else s.max(-1, keepdim=True).values
    e = torch.exp(s - mx)
    den = e.sum(-1, keepdim=True)
    if sink is not None:
        den = den + torch.exp(sink - mx)
    return e / den


def latent_attention_mixer(h, p, m, eps, rnd=identity, rows=None, use_sink=True):
    """h [T, W] -> [T, W].  `rows`: (c, kr) of the layer this one reads, or None to form its own."""
    T = h.shape[0]
    H, dim, rd, vd = m["heads"], m["dim"], m["rot_dim"], m["vdim"]
    pos = torch.arange(T)
    cq = rnd(rms_norm(rnd(h @ p["dq"].T), p["dq.norm"], eps))
    q = rnd(cq @ p["uq"].T).reshape(T, H, dim + rd)
    qn = q[..., :dim]
    qr = rnd(rotate_pairs(q[..., dim:], pos, m["rot"]["dims"], m["rot"]["base"]))
    c, kr = rows if rows is not None else latent_rows(h, p, m, eps, rnd)
    k = rnd(c @ p["uk"].T).reshape(T, H, dim)
    v = rnd(c @ p["uv"].T).reshape(T, H, vd)
    mask = torch.tril(torch.ones(T, T, dtype=torch.bool))
    heads = []
    for i in range(H):
        s = (qn[:, i] @ k[:, i].T + qr[:, i] @ kr.T) * m["scale"]
        s = s.masked_fill(~mask, float("-inf"))
        pr = sink_softmax(s, p["sink"][i] if use_sink and "sink" in p else None)
        heads.append(pr @ v[:, i])
    o = rnd(torch.cat(heads, dim=-1))
    return o @ p["o"].T


def moe_route(h, wr, b, k):
    """-> (ids [T, k], weights [T, k], logits [T, E]); ties go to the lower index."""
    z = h @ wr.T + b
    order = torch.sort(z, dim=-1, descending=True, stable=True).indices[:, :k]
    zc = torch.gather(z, 1, order)
    return order, torch.softmax(zc, dim=-1), z


def expert(h, wg, wu, wd, limit, rnd=identity):
    g = torch.clamp(h @ wg.T, max=limit)
    u = torch.clamp(h @ wu.T, min=-limit, max=limit)
    return rnd(g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ wd.T


def moe(h, p, f, rnd=identity, margins: list | None = None):
    E, k, limit = f["router"]["experts"], f["router"]["top"], f["expert"]["limit"]
    ids, w, z = moe_route(h, p["router"], p["router.b"], k)
    if margins is not None:
        zs = torch.sort(z, dim=-1, descending=True).values
        margins.append(zs[:, k - 1] - zs[:, k] if E > k else torch.full((h.shape[0],), float("inf"), dtype=h.dtype))
    out = torch.zeros_like(h)
    for e in range(E):
        for j in range(k):
            sel = ids[:, j] == e
            if sel.any():
                out[sel] += w[sel, j:j + 1] * expert(h[sel], p[f"e{e}.gate"], p[f"e{e}.up"], p[f"e{e}.down"], limit, rnd)
    return out


def sub(t: dict, prefix: str) -> dict:
    return {n[len(prefix):]: v for n, v in t.items() if n.startswith(prefix)}


def forward(cfg, t, tokens, rnd=identity, streams: list | None = None, margins: list | None = None):
    """Logits [T, vocab] of a whole sequence; `streams` collects the residual stream after every layer,
    `margins` per routed layer the gap between the last chosen and the first rejected router logit."""
    eps = cfg["norm"]["eps"]
    x = t["embed"][torch.as_tensor(tokens, dtype=torch.long)] * cfg["embedding"]["scale"]
    rows = {}
    for i, spec in enumerate(cfg["layers"]):
        m = spec["mixer"]
        h = rnd(layer_norm(x, t[f"l{i}.norm1"], eps))
        p = sub(t, f"l{i}.mix.")
        src = m.get("kv_from")
        if src is None:
            rows[i] = latent_rows(h, p, m, eps, rnd)
        y = latent_attention_mixer(h, p, m, eps, rnd, rows=rows[i if src is None else src])
        if spec.get("mlp") is not None:
            y = y + moe(h, sub(t, f"l{i}.mlp."), spec["mlp"], rnd, margins)
        x = x + cfg["residual_mult"] * y
        if streams is not None:
            streams.append(x.clone())
    return rnd(layer_norm(x, t["final.norm"], eps)) @ t["embed"].T
