"""Small Lenesun configurations for the tests.  They differ from one another in every size and
constant: width, vocabulary, eps, the stream's multiplier and the embedding's scale (also 1), head
counts (1 to 10), unrotated, rotated and value sizes per head (all different, not multiples of 32,
one without a multiple of 8 anywhere), latent sizes (up to 160), which layers read another layer's
cached rows, which layers have experts, expert counts and how many are chosen (one, some, all)."""


def lat(heads, dim, rot_dim, vdim, q_rank, kv_rank, scale, base, kv_from=None, rot_dims=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank,
         "scale": scale, "rot": {"dims": rot_dim if rot_dims is None else rot_dims, "base": base}}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


def moe(experts, top, ff, limit):
    return {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff, "limit": limit}}


def layer(mixer, mlp):
    return {"type": "latent_attention", "mixer": mixer, "mlp": mlp}


L_A = {
    "architecture": "Lenesun", "vocab": 200, "width": 64, "norm": {"eps": 1e-6}, "residual_mult": 0.7,
    "embedding": {"scale": 2.0},
    "layers": [
        layer(lat(2, 16, 8, 24, 24, 32, 0.2, 10000.0), moe(4, 2, 32, 1.0)),
        layer(lat(3, 8, 8, 16, 16, 32, 0.3, 10000.0, kv_from=0), None),
        layer(lat(1, 32, 16, 8, 40, 48, 0.15, 500.0), moe(3, 1, 48, 2.5)),
        layer(lat(2, 24, 16, 32, 8, 48, 0.25, 500.0, kv_from=2), moe(5, 3, 16, 0.5)),
    ],
}

# ten heads (more than one chunk of heads per block), every expert chosen
L_B = {
    "architecture": "Lenesun", "vocab": 150, "width": 96, "norm": {"eps": 1e-5}, "residual_mult": 0.35,
    "embedding": {"scale": 5.5},
    "layers": [
        layer(lat(10, 16, 32, 8, 48, 64, 0.18, 200000.0), moe(8, 8, 16, 3.0)),
        layer(lat(4, 32, 32, 48, 64, 64, 0.1, 200000.0, kv_from=0), moe(2, 1, 64, 1.25)),
    ],
}

# no size a multiple of 8: the plain bfloat16 products and unaligned cache rows
L_C = {
    "architecture": "Lenesun", "vocab": 101, "width": 36, "norm": {"eps": 1e-5}, "residual_mult": 1.0,
    "embedding": {"scale": 1.0},
    "layers": [
        layer(lat(3, 12, 6, 10, 20, 28, 0.22, 3000.0), moe(3, 2, 18, 1.5)),
        layer(lat(2, 10, 6, 14, 12, 28, 0.3, 3000.0, kv_from=0), None),
        layer(lat(1, 20, 10, 6, 14, 22, 0.2, 900.0), moe(6, 1, 10, 0.75)),
    ],
}

# a latent wider than 128 and heads of 64
L_D = {
    "architecture": "Lenesun", "vocab": 320, "width": 128, "norm": {"eps": 1e-4}, "residual_mult": 0.5,
    "embedding": {"scale": 0.5},
    "layers": [
        layer(lat(4, 64, 64, 64, 96, 160, 0.08, 1e6), None),
        layer(lat(2, 64, 64, 32, 32, 160, 0.09, 1e6, kv_from=0), moe(4, 2, 128, 7.0)),
    ],
}

# one layer, one head, no experts anywhere
L_E = {
    "architecture": "Lenesun", "vocab": 64, "width": 48, "norm": {"eps": 1e-5}, "residual_mult": 1.5,
    "embedding": {"scale": 3.5},
    "layers": [layer(lat(1, 48, 16, 40, 32, 24, 0.12, 10000.0), None)],
}

ALL = {"A": L_A, "B": L_B, "C": L_C, "D": L_D, "E": L_E}
