"""Small Zekivik configurations for the tests.  They differ from one another in every size and
constant: width, vocabulary, eps, layer order, which layers have a feed-forward, head counts and
grouping, key and value head sizes (equal, smaller, larger, not multiples of 32), taps (1 to 5),
scale, rotated part of the head (none, part, all), decays (0, 1 and between), and the loop (none,
inside the stack, over all of it, a single pass); one has no size that is a multiple of 8."""


def att(heads, kv_heads, dim, vdim, conv, scale, rot_dims, base):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv, "scale": scale,
            "rot": {"dims": rot_dims, "base": base}}


def ret(heads, dim, vdim, decay, rot_dims, base):
    return {"heads": heads, "dim": dim, "vdim": vdim, "decay": decay, "rot": {"dims": rot_dims, "base": base}}


def dense(ff):
    return {"kind": "dense", "ff": ff}


Z_A = {
    "architecture": "Zekivik", "vocab": 200, "width": 64, "norm": {"eps": 1e-6},
    "layers": [
        {"type": "retention", "mixer": ret(2, 16, 24, [0.9, 0.99], 8, 10000.0), "mlp": dense(96)},
        {"type": "attention", "mixer": att(4, 2, 32, 16, 3, 0.2, 16, 50000.0), "mlp": None},
        {"type": "retention", "mixer": ret(1, 48, 16, [1.0], 48, 300.0), "mlp": None},
        {"type": "attention", "mixer": att(2, 1, 16, 48, 2, 0.3, 16, 1000.0), "mlp": dense(40)},
    ],
    "loop": {"start": 1, "stop": 3, "times": 2},
}

# key and value heads of 64: the tensor-core attention kernels run in bfloat16
Z_B = {
    "architecture": "Zekivik", "vocab": 150, "width": 72, "norm": {"eps": 1e-5},
    "layers": [
        {"type": "attention", "mixer": att(3, 3, 64, 64, 5, 0.125, 64, 200000.0), "mlp": dense(48)},
        {"type": "retention", "mixer": ret(3, 32, 64, [0.5, 0.97, 0.0], 32, 7000.0), "mlp": dense(64)},
    ],
}

# everything looped, one tap, four query heads on one key/value head, heads of 128
Z_C = {
    "architecture": "Zekivik", "vocab": 320, "width": 96, "norm": {"eps": 1e-5},
    "layers": [
        {"type": "attention", "mixer": att(4, 1, 128, 128, 1, 0.09, 32, 1e6), "mlp": None},
        {"type": "retention", "mixer": ret(2, 64, 128, [0.999, 0.75], 16, 500.0), "mlp": dense(80)},
    ],
    "loop": {"start": 0, "stop": 2, "times": 3},
}

# sizes that are no multiple of 32, no rotation at all, a loop of a single pass over one layer
Z_D = {
    "architecture": "Zekivik", "vocab": 97, "width": 40, "norm": {"eps": 1e-4},
    "layers": [
        {"type": "retention", "mixer": ret(3, 24, 40, [0.8, 0.9, 0.95], 0, 10000.0), "mlp": None},
        {"type": "attention", "mixer": att(5, 5, 24, 40, 4, 0.25, 0, 10000.0), "mlp": dense(56)},
        {"type": "attention", "mixer": att(2, 2, 96, 32, 2, 0.1, 48, 20000.0), "mlp": None},
    ],
    "loop": {"start": 1, "stop": 2, "times": 1},
}

# no size a multiple of 8: the plain bfloat16 product and the scalar forms of the row kernels
Z_E = {
    "architecture": "Zekivik", "vocab": 101, "width": 36, "norm": {"eps": 1e-5},
    "layers": [
        {"type": "attention", "mixer": att(3, 1, 20, 12, 3, 0.22, 10, 3000.0), "mlp": dense(50)},
        {"type": "retention", "mixer": ret(1, 14, 18, [0.93], 6, 900.0), "mlp": None},
    ],
}

ALL = {"A": Z_A, "B": Z_B, "C": Z_C, "D": Z_D, "E": Z_E}
