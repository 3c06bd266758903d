"""A plain, slow implementation of the Zekivik decoder, for tests only.

Whole sequences, no cache, no batching, one function per mechanism, ordinary tensor
arithmetic (double precision unless told otherwise).  It shares no code with the library.

The design in this file's notation.  A model is a list of layers over a residual stream x
[T, W].  A layer: x += s1 * mixer(n1(x)), and, where the layer has a feed-forward,
x += s2 * ff(n2(x)), with n(x) = x / sqrt(mean(x^2) + eps) * (1 + w) and
s = sigmoid(R n(x) + b) (an element-wise gate on each sublayer's result, read from the
sublayer's own input).  Layers [start, stop) run `times` times in a row with the same
weights; before every pass but the first the embedding output is added to x, and before every
pass (also the first) row t of the `loop.step` table is added.

Mixers:
* retention: q, k (heads x dim) and v (heads x vdim) are projections; q and k are rotated by
  position on the first `rot.dims` dimensions (pairs (i, i + dims/2)), k is then scaled by
  dim^-1/2; per head S_t = decay * S_{t-1} + k_t v_t^T and o_t = S_t^T q_t; o_t is divided by
  its root mean square per head, multiplied by silu(G h) and projected.
* attention: q, k, v are projections, each passed through a causal depthwise convolution over
  time (taps from the tensor's shape), q and k rotated as above and then divided by their root
  mean square per head, v divided by its root mean square per head; softmax attention with
  grouped key/value heads and the configured scale; each head's result is multiplied by the
  sigmoid of one number per head and projected.
Feed-forward: down(gelu_tanh(gate h) * (up h)).

`rnd` is a rounding hook: the identity for the 32-bit path, rounding to bfloat16 where the
library's bfloat16 path stores a value in bfloat16.
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
        elif e["dtype"] == "I32":
            ten = torch.from_numpy(np.frombuffer(data[b:t], dtype=np.int32).reshape(e["shape"]).copy())
            out[name] = ten
            continue
        else:
            raise ValueError(f"{name}: dtype {e['dtype']}")
        out[name] = ten.to(dtype)
    return out


def identity(t):
    return t


def round_bf16(t):
    return t.to(torch.float32).to(torch.bfloat16).to(t.dtype)


# ---- mechanisms, one function each ---------------------------------------------------------------
def unit_rms(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def offset_norm(x, w, eps):
    """The layer norm: unit_rms(x) * (1 + w), the weight being stored around zero."""
    return unit_rms(x, eps) * (1.0 + w)


def sigmoid(z):
    return 1.0 / (1.0 + torch.exp(-z))


def silu(z):
    return z * sigmoid(z)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def rotate(u, pos, dims, base):
    """u [T, heads, d]; rotates the first `dims` dimensions, pairing i with i + dims/2;
    angle = pos * base^(-2i/dims)."""
    half = dims // 2
    i = torch.arange(half, dtype=u.dtype)
    ang = pos.to(u.dtype)[:, None] * torch.pow(torch.tensor(base, dtype=u.dtype), -2.0 * i / dims)[None, :]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    a, b = u[..., :half], u[..., half:dims]
    out = u.clone()
    out[..., :half] = a * c - b * s
    out[..., half:dims] = b * c + a * s
    return out


def causal_conv(u, w):
    """u [T, C], w [C, taps]: y_t = sum_j w[:, j] * u_{t - taps + 1 + j}, zeros before the start."""
    T, C = u.shape
    taps = w.shape[1]
    pad = torch.cat([torch.zeros(taps - 1, C, dtype=u.dtype), u], 0)
    y = torch.zeros_like(u)
    for j in range(taps):
        y = y + pad[j:j + T] * w[:, j][None, :]
    return y


def retention_scan(q, k, v, decay):
    """q, k [T, H, d], v [T, H, e], decay [H]: S_t = decay S_{t-1} + k_t v_t^T, o_t = S_t^T q_t."""
    T, H, d = q.shape
    e = v.shape[-1]
    S = torch.zeros(H, d, e, dtype=q.dtype)
    o = torch.zeros(T, H, e, dtype=q.dtype)
    for t in range(T):
        S = decay[:, None, None] * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hde,hd->he", S, q[t])
    return o


def retention_mixer(h, p, m, eps, rnd=identity):
    """h [T, W]; p: the mixer's tensors by short name; m: the layer's 'mixer' config."""
    T = h.shape[0]
    H, d, e = m["heads"], m["dim"], m["vdim"]
    pos = torch.arange(T)
    q = rnd(h @ p["q"].T).view(T, H, d)
    k = rnd(h @ p["k"].T).view(T, H, d)
    v = rnd(h @ p["v"].T).view(T, H, e)
    g = rnd(h @ p["g"].T)
    q = rotate(q, pos, m["rot"]["dims"], m["rot"]["base"])
    k = rotate(k, pos, m["rot"]["dims"], m["rot"]["base"]) * d ** -0.5
    o = retention_scan(q, k, v, torch.tensor(m["decay"], dtype=h.dtype))
    o = unit_rms(o, eps).reshape(T, H * e)
    return rnd(o * silu(g)) @ p["o"].T


def softmax_attention(q, k, v, scale, groups):
    """q [T, H, d], k [T, G, d], v [T, G, e]; query head i uses key/value head i // groups."""
    T, H, _ = q.shape
    out = torch.zeros(T, H, v.shape[-1], dtype=q.dtype)
    mask = torch.ones(T, T, dtype=torch.bool).tril()
    for i in range(H):
        sc = (q[:, i] @ k[:, i // groups].T) * scale
        sc = sc.masked_fill(~mask, float("-inf"))
        out[:, i] = torch.softmax(sc, -1) @ v[:, i // groups]
    return out


def attention_mixer(h, p, m, eps, rnd=identity):
    T = h.shape[0]
    H, G, d, e = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    pos = torch.arange(T)
    q = rnd(causal_conv(rnd(h @ p["q"].T), p["q.conv"])).view(T, H, d)
    k = rnd(causal_conv(rnd(h @ p["k"].T), p["k.conv"])).view(T, G, d)
    v = rnd(causal_conv(rnd(h @ p["v"].T), p["v.conv"])).view(T, G, e)
    gate = sigmoid(rnd(h @ p["g"].T))                                   # [T, H]
    q = rnd(unit_rms(rotate(q, pos, m["rot"]["dims"], m["rot"]["base"]), eps))
    k = rnd(unit_rms(rotate(k, pos, m["rot"]["dims"], m["rot"]["base"]), eps))
    v = rnd(unit_rms(v, eps))
    o = softmax_attention(q, k, v, m["scale"], H // G) * gate[:, :, None]
    return rnd(o.reshape(T, H * e)) @ p["o"].T


def dense_ff(h, p, rnd=identity):
    return rnd(gelu_tanh(h @ p["gate"].T) * (h @ p["up"].T)) @ p["down"].T


def sub(t: dict, prefix: str) -> dict:
    return {k[len(prefix):]: v for k, v in t.items() if k.startswith(prefix)}


def layer(x, t, i, spec, eps, rnd=identity):
    """One run of layer i on the residual stream x [T, W]."""
    pre = f"l{i}."
    h = rnd(offset_norm(x, t[pre + "norm1"], eps))
    mix = {"retention": retention_mixer, "attention": attention_mixer}[spec["type"]]
    y = mix(h, sub(t, pre + "mix."), spec["mixer"], eps, rnd)
    x = x + sigmoid(h @ t[pre + "rg1"].T + t[pre + "rg1.b"]) * y
    if spec.get("mlp") is not None:
        assert spec["mlp"]["kind"] == "dense"
        h = rnd(offset_norm(x, t[pre + "norm2"], eps))
        y = dense_ff(h, sub(t, pre + "mlp."), rnd)
        x = x + sigmoid(h @ t[pre + "rg2"].T + t[pre + "rg2.b"]) * y
    return x


def schedule(cfg) -> list[tuple[int, int | None]]:
    """(layer, pass number if the run opens a pass of the loop else None), in running order."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return [(i, None) for i in range(n)]
    a, b, times = loop["start"], loop["stop"], loop["times"]
    runs = [(i, None) for i in range(a)]
    for t in range(times):
        runs += [(i, t if i == a else None) for i in range(a, b)]
    return runs + [(i, None) for i in range(b, n)]


def forward(cfg, t, tokens, rnd=identity, streams: list | None = None):
    """Logits [T, vocab] of one whole sequence.  `streams`, if a list, receives x after every layer run."""
    dt = t["embed"].dtype
    eps = cfg["norm"]["eps"]
    x0 = t["embed"][torch.as_tensor(tokens, dtype=torch.long)]
    x = x0.clone()
    for i, opens in schedule(cfg):
        if opens is not None:
            if opens > 0:
                x = x + x0
            x = x + t["loop.step"][opens]
        x = layer(x, t, i, cfg["layers"][i], eps, rnd)
        if streams is not None:
            streams.append(x.clone())
    xn = rnd(offset_norm(x, t["final.norm"], eps))
    return (xn @ t["head"].T).to(dt)
