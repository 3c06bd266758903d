"""The Lenesun decoder on the GPU against the plain implementation (tests/plain_lenesun.py): every
mechanism alone, then whole models: prompts whole, in portions and token by token, unequal batches,
slots and pages used again, long decoding, and greedy generation through the entry point."""
import os

import numpy as np
import pytest
import torch

import harness as H
import plain_lenesun as P
from lenesun_configs import ALL, lat

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}
TOL = {"float32": H.TOL_F32, "bfloat16": H.TOL_BF16}


def K():
    from lastengine_b200.ops import kernels
    return kernels


def rnd_of(dtype):
    return P.round_bf16 if dtype == "bfloat16" else P.identity


def inputs(T, D, seed, bf16, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    h = torch.randn(T, D, generator=g, dtype=torch.float64) * scale
    return P.round_bf16(h) if bf16 else h


# ---- the small kernels ---------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("M,D", [(1, 36), (5, 64), (70, 200), (3, 2304)])
def test_layer_norm_scaled_sum_and_scaled_embedding(M, D, dtype):
    k = K()
    x = inputs(M, D, 1, False, 3.0) + 1.7            # a mean well away from zero
    y = inputs(M, D, 2, False)
    w = 1.0 + 0.3 * inputs(1, D, 3, False)[0]
    eps = 1e-3
    out = torch.zeros(M, D, dtype=DT[dtype], device=DEV)
    k.layernorm(out, x.to(DEV, torch.float32), w.to(DEV, torch.float32), eps)
    assert H.rel_err(out, P.layer_norm(x, w, eps)) < (1e-5 if dtype == "float32" else 5e-3)
    rows = torch.tensor([M - 1, 0], dtype=torch.int32, device=DEV)
    out2 = torch.zeros(2, D, dtype=DT[dtype], device=DEV)
    k.layernorm(out2, x.to(DEV, torch.float32), w.to(DEV, torch.float32), eps, rows=rows)
    assert H.rel_err(out2, P.layer_norm(x[[M - 1, 0]], w, eps)) < (1e-5 if dtype == "float32" else 5e-3)
    # x += m * y, alone and with the norm of the new rows
    xs = x.to(DEV, torch.float32)
    k.scaled_residual(xs, y.to(DEV, torch.float32), 0.35)
    assert H.rel_err(xs, x + 0.35 * y) < 1e-6
    xs = x.to(DEV, torch.float32)
    h = torch.zeros(M, D, dtype=DT[dtype], device=DEV)
    k.scaled_residual(xs, y.to(DEV, torch.float32), -1.5, h=h, norm_w=w.to(DEV, torch.float32), eps=eps)
    assert H.rel_err(xs, x - 1.5 * y) < 1e-6
    assert H.rel_err(h, P.layer_norm(x - 1.5 * y, w, eps)) < (1e-5 if dtype == "float32" else 5e-3)
    # the embedding row times a constant; the table stays as it is
    table = P.round_bf16(inputs(11, D, 4, False))
    toks = torch.tensor([10, 0, 3][:max(1, min(3, M))], dtype=torch.int32, device=DEV)
    e = torch.zeros(toks.numel(), D, dtype=torch.float32, device=DEV)
    k.embed(e, table.to(DEV, DT[dtype]), toks, 2.5)
    assert H.rel_err(e, table[toks.cpu().long()] * 2.5) < 1e-6


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("M,D,E,k", [(1, 64, 4, 2), (9, 36, 3, 1), (300, 96, 8, 8), (33, 128, 40, 5)])
def test_router_chooses_by_logit_and_weighs_by_softmax_over_the_chosen(M, D, E, k, dtype):
    kk = K()
    bf16 = dtype == "bfloat16"
    h = inputs(M, D, 5, bf16)
    wr = P.round_bf16(inputs(E, D, 6, False, 0.4))
    b = inputs(1, E, 7, False, 2.0)[0].float().double()     # biases large enough to change the choice
    ids = torch.zeros(M, k, dtype=torch.int32, device=DEV)
    wts = torch.zeros(M, k, dtype=torch.float32, device=DEV)
    kk.moe_router(ids, wts, h.to(DEV, DT[dtype]), wr.to(DEV, torch.float32), b.to(DEV, torch.float32), True, 1.0,
                  softmax_chosen=True)
    wi, ww, z = P.moe_route(h, wr, b, k)
    wi0, _, _ = P.moe_route(h, wr, torch.zeros_like(b), k)
    if M >= 30:
        assert not torch.equal(wi, wi0)                    # the bias is part of what is compared
    zs = torch.sort(z, dim=-1, descending=True).values
    sure = (zs[:, :-1] - zs[:, 1:]).amin(-1) > 1e-4 if E > 1 else torch.ones(M, dtype=torch.bool)
    assert sure.float().mean() > 0.7
    assert torch.equal(ids.cpu().long()[sure], wi[sure])
    assert (wts.cpu().double()[sure] - ww[sure]).abs().max() < 1e-5
    assert (wts.sum(-1) - 1).abs().max() < 1e-5


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_clamped_expert_activation(dtype):
    kk = K()
    M, F = 7, 24
    gu = inputs(M, 2 * F, 8, False, 3.0)                   # many values beyond the limit on both sides
    out = torch.zeros(M, F, dtype=DT[dtype], device=DEV)
    kk.gated_act(out, gu.to(DEV, torch.float32), kk.CLAMPED_SIGMOID, 1.25, 1.702)
    g = torch.clamp(gu[:, :F], max=1.25)
    u = torch.clamp(gu[:, F:], -1.25, 1.25)
    want = g * torch.sigmoid(1.702 * g) * (u + 1)
    assert (gu[:, :F] < -1.25).any() and (gu[:, :F] > 1.25).any()      # the gate is clamped from above only
    assert H.rel_err(out, want) < (1e-6 if dtype == "float32" else 5e-3)


@pytest.mark.parametrize("M,Kd,F", [(1, 64, 48), (8, 96, 160), (16, 256, 512), (40, 128, 256), (128, 256, 2048),
                                   (300, 64, 96), (700, 512, 1024), (1100, 256, 4096)])
def test_clamped_activation_as_the_epilogue_of_every_bfloat16_product(M, Kd, F):
    """Rows from one to over a thousand reach the weight stream, the sliced and the tiled tensor-core products
    and the one on pairs of SMs; each clamps, applies g sigmoid(1.702 g) (u + 1) and stores."""
    from lastengine_b200.parts.ffn import fuse_gate_up
    kk = K()
    g = torch.Generator().manual_seed(M)
    x = P.round_bf16(torch.randn(M, Kd, generator=g, dtype=torch.float64))
    wg = P.round_bf16(torch.randn(F, Kd, generator=g, dtype=torch.float64) * (2.0 / Kd ** 0.5))
    wu = P.round_bf16(torch.randn(F, Kd, generator=g, dtype=torch.float64) * (2.0 / Kd ** 0.5))
    w = fuse_gate_up(wg.to(DEV, torch.bfloat16), wu.to(DEV, torch.bfloat16), True)
    for limit in (1.5, 0.75):
        epi = kk.gated_epilogue(kk.CLAMPED_SIGMOID, limit, 1.702)
        assert epi is not None
        gt = torch.clamp(x @ wg.T, max=limit)
        up = torch.clamp(x @ wu.T, -limit, limit)
        want = gt * torch.sigmoid(1.702 * gt) * (up + 1)
        assert ((x @ wg.T) > limit).any() and ((x @ wu.T) < -limit).any()
        for dt, tol in ((torch.bfloat16, 8e-3), (torch.float32, 3e-4)):
            out = torch.zeros(M, F, dtype=dt, device=DEV)
            kk.linear(out, x.to(DEV, torch.bfloat16), w, epi)
            kk.check_device_status()
            assert H.rel_err(out, want) < tol
    # no fused form for a limit bfloat16 does not hold, or another slope: the part then runs the kernel of its own
    assert kk.gated_epilogue(kk.CLAMPED_SIGMOID, 1.3, 1.702) is None and kk.gated_epilogue(kk.CLAMPED_SIGMOID, 1.5, 1.0) is None


def test_grouped_clamped_epilogue_equals_the_unfused_path():
    """The expert layer with the fused epilogue (limit 1.5) and with the kernel of its own (limit 1.3) against
    the plain experts, for a prompt's rows and a decode step's."""
    from lastengine_b200.engine.workspace import Workspace
    from lastengine_b200.parts.base import BuildEnv
    from lastengine_b200.registry import FEED_FORWARDS
    from lastengine_b200.weights.random_init import random_tensor
    D, E, k, F = 64, 6, 2, 48
    for limit, fused in ((1.5, True), (1.3, False)):
        names = {"router": "router", "bias": "router.b", "gate": "e{e}.gate", "up": "e{e}.up", "down": "e{e}.down"}
        part = FEED_FORWARDS.get("topk_moe")(hidden_size=D, num_experts=E, top_k=k, expert_size=F, router="softmax_chosen",
                                             activation="clamped_sigmoid", limit=limit, alpha=1.702, names=names)
        plain_t = {n: random_tensor(n, sp, 3, 0.3).to(torch.bfloat16).double() for n, sp in part.tensors().items()}
        plain_t["router"] = plain_t["router"] * 3.0          # logits well apart
        dev = torch.device(DEV)
        env = BuildEnv(device=dev, dtype=torch.bfloat16, workspace=Workspace(dev))
        from lastengine_b200.weights.loader import kept_dtype
        part.load({n: v.float().to(dev, kept_dtype(part.tensors()[n], torch.bfloat16, torch.bfloat16)) for n, v in plain_t.items()}, env)
        assert part.fused == fused
        f = {"router": {"experts": E, "top": k}, "expert": {"ff": F, "limit": limit}}
        for M in (3, 200):
            h = inputs(M, D, 60 + M, True)
            out = torch.zeros(M, D, dtype=torch.float32, device=DEV)
            part.forward(h.to(DEV, torch.bfloat16), out, False, None, env)
            margins = []
            want = P.moe(h, plain_t, f, P.round_bf16, margins)
            ok = margins[0] > 2e-2
            assert ok.float().mean() > 0.7
            assert H.rel_err(out[ok.to(DEV)], want[ok]) < H.TOL_BF16


# ---- a mixer alone: its own cache, steps laid out as the engine lays them out ----------------------
class MixerRig:
    def __init__(self, params, dtype, seed=0, std=0.3, max_tokens=2048, max_seqs=6, edit=None):
        from lastengine_b200.cache import Cache
        from lastengine_b200.engine.batch import BatchBuilder
        from lastengine_b200.engine.workspace import Workspace
        from lastengine_b200.parts.base import BuildEnv
        from lastengine_b200.registry import MIXERS
        from lastengine_b200.weights.loader import kept_dtype
        from lastengine_b200.weights.random_init import random_tensor
        dev = torch.device(DEV)
        self.env = BuildEnv(device=dev, dtype=DT[dtype], workspace=Workspace(dev))
        self.mixer = MIXERS.get("latent_attention")(**params)
        self.plain = {}
        for name, spec in self.mixer.tensors().items():
            self.plain[name] = random_tensor(name, spec, seed, std, norm_init="random").to(torch.bfloat16).double()
        if edit:
            edit(self.plain)
        self.mixer.load({n: v.float().to(dev, kept_dtype(self.mixer.tensors()[n], torch.bfloat16, DT[dtype]))
                         for n, v in self.plain.items()}, self.env)
        self.cache = Cache({0: self.mixer.cache_spec()}, max_tokens=max_tokens, max_seqs=max_seqs, dtype=DT[dtype], device=dev)
        self.builder = BatchBuilder(dev)
        self.D = params["hidden_size"]

    def step(self, slots, hs, writable=True):
        grow = {s: h.shape[0] for s, h in zip(slots, hs)}
        pos0 = [self.cache.length(s) for s in slots]
        self.cache.reserve(grow)
        tables = {gi: g.table(list(slots), max(1, max(len(g.seq_pages.get(s, ())) for s in slots)))
                  for gi, g in enumerate(self.cache.kv_groups)}
        batch = self.builder.build(list(slots), [[0] * h.shape[0] for h in hs], pos0, [], tables)
        h = torch.cat(hs, 0).to(DEV, self.env.dtype)
        out = torch.zeros(h.shape[0], self.D, dtype=torch.float32, device=DEV)
        self.mixer.forward(h, out, False, batch, self.cache.view(0, writable, batch.tables), self.env)
        K().check_device_status()
        self.cache.commit(grow)
        return list(torch.split(out.double().cpu(), [x.shape[0] for x in hs]))


def lat_params(D, m, sink=True, own_kv=True):
    from lastengine_b200.parts.base import PartSpec
    pos = PartSpec("rope", {"rope_dim": m["rot"]["dims"], "theta": m["rot"]["base"], "style": "adjacent"}) \
        if m["rot"]["dims"] else None
    return dict(hidden_size=D, num_heads=m["heads"], head_dim=m["dim"], rope_dim=m["rot_dim"], v_head_dim=m["vdim"],
                q_rank=m["q_rank"], kv_rank=m["kv_rank"], norm_eps=1e-5, scale=m["scale"], position=pos, sink=sink,
                own_kv=own_kv)


LAT_CASES = [   # heads, dim, rot_dim, vdim, q_rank, kv_rank, scale, rotated dims, sink
    (2, 16, 8, 24, 24, 32, 0.2, 8, True),
    (1, 48, 16, 8, 16, 40, 0.1, 16, False),
    (10, 8, 32, 16, 40, 64, 0.25, 32, True),        # more heads than one block takes
    (3, 12, 6, 10, 20, 28, 0.3, 6, True),           # nothing a multiple of 8
    (5, 24, 16, 40, 32, 72, 0.15, 8, True),         # half of the rotated part passes unrotated
    (4, 64, 64, 64, 96, 160, 0.08, 64, True),
    (2, 32, 8, 16, 48, 288, 0.05, 8, True),         # a latent beyond 256
    (2, 16, 0, 16, 24, 32, 0.2, 0, True),           # no rotated part at all
    (16, 32, 16, 32, 64, 128, 0.1, 16, True),       # four rows of sixteen heads in a tensor-core block
    (6, 16, 32, 24, 48, 96, 0.12, 32, True),        # ten rows of six heads; an odd number of tiles across the latent
    (70, 8, 16, 8, 32, 32, 0.2, 16, True),          # more heads than a tensor-core block takes
]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("case", LAT_CASES)
def test_latent_attention_alone_whole_in_portions_and_batched(case, dtype):
    heads, dim, rd, vd, qr, kr, scale, rot, sink = case
    bf16 = dtype == "bfloat16"
    D = 40
    m = lat(heads, dim, rd, vd, qr, kr, scale, 5000.0, rot_dims=rot)

    def edit(t):
        if sink:
            t["sink"] = P.round_bf16(torch.linspace(-1.0, 2.5, heads, dtype=torch.float64))

    rig = MixerRig(lat_params(D, m, sink=sink), dtype, seed=5, edit=edit)
    rnd = rnd_of(dtype)
    hs = [inputs(n, D, 10 + n, bf16) for n in (150, 1, 37)]
    want = [P.latent_attention_mixer(h, rig.plain, m, 1e-5, rnd) for h in hs]
    if sink:       # the sink is worth a hundred tolerances: a kernel that left it out would not pass
        assert H.rel_err(P.latent_attention_mixer(hs[0], rig.plain, m, 1e-5, use_sink=False), want[0]) > 100 * H.TOL_F32
    tol = TOL[dtype]
    for h, w in zip(hs, want):
        s = rig.cache.alloc_seq()
        got = rig.step([s], [h])[0]
        rig.cache.free_seq(s)
        assert H.rel_err(got, w) < tol
    more = [inputs(21, D, 50 + i, bf16) for i in range(3)]
    want2 = [P.latent_attention_mixer(torch.cat([h, x]), rig.plain, m, 1e-5, rnd) for h, x in zip(hs, more)]
    slots = [rig.cache.alloc_seq() for _ in hs]          # the slots and pages just given back
    got = rig.step(slots, hs)
    for g, w in zip(got, want):
        assert H.rel_err(g, w) < tol
    cuts = [0, 2, 3, 8, 9, 21]
    outs = [[] for _ in hs]
    for a, b in zip(cuts[:-1], cuts[1:]):
        for i, g in enumerate(rig.step(slots, [x[a:b] for x in more])):
            outs[i].append(g)
    for i, w in enumerate(want2):
        assert H.rel_err(torch.cat(outs[i]), w[hs[i].shape[0]:]) < tol, f"sequence {i} after portions"


def test_latent_attention_reaches_a_row_far_back_and_at_page_borders():
    """Weights and inputs made so that the last position's query meets one far cached row with a score
    far above the rest: input channel 0 alone feeds number 0 of the query latent and channel 1 number 0 of
    the key/value latent, and those feed dimension 0 of head 0's unrotated query and key."""
    D = 32
    m = lat(2, 16, 8, 24, 24, 32, 0.2, 5000.0)

    def edit(t):
        for n, up, ch in (("dq", "uq", 0), ("dkv", "uk", 1)):
            t[n][:, :2] = 0.0                       # nothing else reads the two channels
            t[n][0] = 0.0
            t[n][0, ch] = 8.0                       # latent number 0 reads its input channel
            t[up][0] = 0.0
            t[up][0, 0] = 3.0                       # and dimension 0 of head 0 reads latent number 0
        t["dq.norm"][0] = 1.0
        t["dkv.norm"][0] = 1.0

    for far in (3, 63, 64, 65, 127, 128, 500):
        rig = MixerRig(lat_params(D, m), "float32", seed=9, std=0.1, edit=edit)
        T = 700
        h = inputs(T, D, 4, False) * 0.3
        h[:, :2] = 0.0
        h[far, 1] = 30.0
        h[T - 1, 0] = 30.0
        want = P.latent_attention_mixer(h, rig.plain, m, 1e-5)
        cut = torch.cat([h[:far], h[far + 1:]])
        assert H.rel_err(P.latent_attention_mixer(cut, rig.plain, m, 1e-5)[-1:], want[-1:]) > 0.02      # a thousand tolerances
        s = rig.cache.alloc_seq()
        whole = rig.step([s], [h])[0]
        rig.cache.free_seq(s)
        assert H.rel_err(whole, want) < H.TOL_F32
        s = rig.cache.alloc_seq()
        head = rig.step([s], [h[:T - 3]])[0]
        tail = torch.cat([rig.step([s], [h[i:i + 1]])[0] for i in range(T - 3, T)])
        assert H.rel_err(torch.cat([head, tail]), want) < H.TOL_F32, f"far row at {far}"


def test_tensor_core_and_general_latent_attention_agree():
    """bfloat16: the same steps through the tensor-core kernel and through the general one."""
    D = 64
    m = lat(5, 16, 16, 24, 32, 64, 0.2, 5000.0)
    hs = [inputs(n, D, 30 + n, True) for n in (200, 70, 1)]
    outs = {}
    assert K().latent_attention_uses_mma(torch.bfloat16, 64, 16, 64, 64)
    assert not K().latent_attention_uses_mma(torch.float32, 64, 16, 64, 64)
    assert not K().latent_attention_uses_mma(torch.bfloat16, 72, 16, 64, 72)
    try:
        for on in (True, False):
            K().set_latent_mma(on)
            rig = MixerRig(lat_params(D, m), "bfloat16", seed=4)
            slots = [rig.cache.alloc_seq() for _ in hs]
            got = rig.step(slots, [h[:-2] if h.shape[0] > 2 else h for h in hs])
            tails = [rig.step(slots[:2], [h[i:i + 1] for h in hs[:2]]) for i in (-2, -1)]
            outs[on] = torch.cat(got + [t for pair in tails for t in pair])
    finally:
        K().set_latent_mma(True)
    want = torch.cat([P.latent_attention_mixer(h, rig.plain, m, 1e-5, P.round_bf16) for h in hs])
    assert H.rel_err(outs[True], outs[False]) < H.TOL_BF16 / 3
    assert H.rel_err(outs[True][:198], want[:198]) < H.TOL_BF16


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_decoding_with_the_key_range_cut_into_pieces_for_the_blocks(dtype):
    """One row per sequence and long sequences: the kernel cuts the cached rows into pieces, and the
    pieces' sums meet the sink in the merge."""
    bf16 = dtype == "bfloat16"
    D = 48
    m = lat(3, 16, 16, 24, 24, 64, 0.2, 5000.0)
    rig = MixerRig(lat_params(D, m), dtype, seed=3, max_tokens=4096,
                   edit=lambda t: t.__setitem__("sink", torch.tensor([1.5, -0.5, 3.0], dtype=torch.float64)))
    hs = [inputs(n, D, 20 + n, bf16) for n in (1500, 700)]
    want = [P.latent_attention_mixer(h, rig.plain, m, 1e-5, rnd_of(dtype)) for h in hs]
    slots = [rig.cache.alloc_seq() for _ in hs]
    rig.step(slots, [h[:-4] for h in hs])
    got = [[], []]
    for i in range(4, 0, -1):
        out = rig.step(slots, [h[h.shape[0] - i: h.shape[0] - i + 1] for h in hs])
        for j in range(2):
            got[j].append(out[j])
    for j in range(2):
        assert H.rel_err(torch.cat(got[j]), want[j][-4:]) < TOL[dtype]


def test_a_layer_reads_the_rows_another_layer_cached():
    D = 40
    m0 = lat(2, 16, 8, 24, 24, 32, 0.2, 5000.0)
    m1 = lat(3, 8, 8, 16, 16, 32, 0.3, 5000.0, kv_from=0)
    a = MixerRig(lat_params(D, m0), "float32", seed=1)
    b = MixerRig(lat_params(D, m1, own_kv=False), "float32", seed=2)
    assert "dkv" not in b.plain and "dkv.norm" not in b.plain
    b.cache, b.builder = a.cache, a.builder           # one cache entry, written by a, read by b
    h0, h1 = inputs(90, D, 1, False), inputs(90, D, 2, False)
    rows = P.latent_rows(h0, a.plain, m0, 1e-5)
    want = P.latent_attention_mixer(h1, b.plain, m1, 1e-5, rows=rows)
    s = a.cache.alloc_seq()
    outs = []
    for lo, hi in ((0, 70), (70, 71), (71, 90)):
        a.step([s], [h0[lo:hi]])
        # the reader's step covers the same positions: the rows are there, the lengths are put back for it
        a.cache.lens[s] -= hi - lo
        outs.append(b.step([s], [h1[lo:hi]], writable=False)[0])
    assert H.rel_err(torch.cat(outs), want) < H.TOL_F32


# ---- whole models --------------------------------------------------------------------------------
@pytest.fixture(scope="module")
def dirs(tmp_path_factory):
    from lastengine_b200.weights import write_model_dir
    return {n: write_model_dir(cfg, str(tmp_path_factory.mktemp("l" + n)), seed=21 + i, norm_init="random")
            for i, (n, cfg) in enumerate(ALL.items())}


_plain = {}


def plain(name, dirs, tokens, bf16):
    """(logits, positions whose routing does not hang on rounding)"""
    key = (name, tuple(tokens), bf16)
    if key not in _plain:
        t = P.read_safetensors(os.path.join(dirs[name], "model.safetensors"))
        margins = []
        lg = P.forward(ALL[name], t, tokens, rnd=rnd_of("bfloat16" if bf16 else "float32"), margins=margins)
        gap = torch.stack(margins).amin(0) if margins else torch.full((len(tokens),), float("inf"), dtype=torch.float64)
        # a flipped choice also changes what every later position attends to
        ok = torch.cummin((gap > (2e-2 if bf16 else 1e-5)).to(torch.int8), 0).values.bool()
        _plain[key] = (lg, ok)
    return _plain[key]


def close(got, wanted, dtype) -> bool:
    """32-bit: every position within the tolerance.  bfloat16: the two computations round at different
    places (the library never forms a head's keys), so they are compared over the positions whose
    routing is decided: half within a third of the tolerance, nine in ten within it."""
    want, ok = wanted
    if dtype == "float32":
        assert ok.float().mean() > 0.9
        return H.rel_err(got[ok], want[ok]) < H.TOL_F32
    want = want.double()
    e = (got.double().cpu() - want).abs().amax(dim=-1) / want.abs().max()
    e = e[ok]
    if e.numel() < 8:
        return bool(e.numel() == 0 or e.max() < 3 * H.TOL_BF16)
    return bool(e.median() < H.TOL_BF16 / 3 and torch.quantile(e, 0.9) < H.TOL_BF16)


def reqs_for(name, lengths, seed):
    rng = np.random.default_rng(seed)
    return [rng.integers(0, ALL[name]["vocab"], size=n).tolist() for n in lengths]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(ALL))
def test_model_whole_tail_portions_and_batches(name, dtype, dirs):
    from lastengine_b200 import Engine
    bf16 = dtype == "bfloat16"
    eng = Engine.from_pretrained(dirs[name], dtype=dtype, max_tokens=1024, max_seqs=6)
    reqs = reqs_for(name, [150, 3, 70, 1], 40)
    want = [plain(name, dirs, r, bf16) for r in reqs]
    for r, w in zip(reqs, want):
        assert close(H.run_whole(eng, r), w, dtype), f"whole, {len(r)} tokens"
    assert close(H.run_tail(eng, reqs[0], tail=90), want[0], dtype)          # decoding across a page border
    assert close(H.run_tail(eng, reqs[2], tail=69), want[2], dtype)          # from the first token on
    s = eng.new_sequence()
    outs, at = [], 0
    for n in (2, 1, 2, 59, 1, 64, 3, 18):
        outs.append(H.to_host(eng.step([s], [reqs[0][at:at + n]], [list(range(n))], check=True)))
        at += n
    eng.release(s)
    assert at == 150 and close(torch.cat(outs), want[0], dtype)
    got = H.run_batch(eng, reqs, [100, 1, 64, 1])
    for g, w, r in zip(got, want, reqs):
        assert close(g, w, dtype), f"batched, {len(r)} tokens"
    got = H.run_batch(eng, reqs[::-1], [1, 7, 2, 149])          # the slots and pages just given back, in another order
    for g, w in zip(got, want[::-1]):
        assert close(g, w, dtype)
    assert eng.cache.slots.n_held == 0
    eng.cache.check()


def test_the_stream_after_every_layer_in_32_bit(dirs):
    """Layer by layer: the residual stream of a one-layer and a two-layer cut of a model equals the plain
    implementation's stream after those layers (the final norm and the head are undone by comparing logits
    of models that end there)."""
    import copy
    from lastengine_b200 import Engine
    from lastengine_b200.weights import write_model_dir  # noqa: F401
    name = "A"
    t = P.read_safetensors(os.path.join(dirs[name], "model.safetensors"))
    toks = reqs_for(name, [80], 46)[0]
    for n_layers in (1, 2, 3, 4):
        cfg = copy.deepcopy(ALL[name])
        cfg["layers"] = cfg["layers"][:n_layers]
        eng = Engine(__import__("lastengine_b200.registry", fromlist=["x"]).plan_from_config(cfg), dtype="float32", max_tokens=256)
        from lastengine_b200.weights.loader import kept_dtype
        specs = eng.model.tensor_specs()
        alias = eng.plan.tensor_aliases
        eng.model.load({alias(k): v.float().to(DEV, kept_dtype(specs[alias(k)], torch.bfloat16, torch.float32))
                        for k, v in t.items() if alias(k) in specs})
        eng.loaded = True
        assert H.rel_err(H.run_whole(eng, toks), P.forward(cfg, t, toks)) < H.TOL_F32, f"{n_layers} layers"


@pytest.mark.parametrize("name", ["A", "C"])
def test_logits_do_not_depend_on_the_cut_or_the_batch_beyond_rounding(name, dirs):
    from lastengine_b200 import Engine
    eng = Engine.from_pretrained(dirs[name], dtype="float32", max_tokens=1024, max_seqs=6)
    reqs = reqs_for(name, [140, 9], 41)
    whole = H.run_whole(eng, reqs[0])
    tail = H.run_tail(eng, reqs[0], tail=80)
    batched = H.run_batch(eng, reqs, [61, 4])[0]
    assert H.rel_err(tail, whole) < 5e-6 and H.rel_err(batched, whole) < 5e-6


@pytest.mark.parametrize("name,dtype", [("A", "float32"), ("D", "float32"), ("B", "bfloat16")])
def test_long_decoding_from_a_short_prompt(name, dtype, dirs):
    from lastengine_b200 import Engine
    eng = Engine.from_pretrained(dirs[name], dtype=dtype, max_tokens=512, max_seqs=2)
    r = reqs_for(name, [200], 42)[0]
    got = H.run_tail(eng, r, tail=196)
    assert close(got, plain(name, dirs, r, dtype == "bfloat16"), dtype)


def plain_greedy(name, dirs, prompt, n, bf16):
    toks, out, margins = list(prompt), [], []
    for _ in range(n):
        lg, ok = plain(name, dirs, toks, bf16)
        lg = lg[-1]
        top = torch.topk(lg, 2).values
        margins.append(float((top[0] - top[1]) / lg.abs().max()) if bool(ok[-1]) else 0.0)
        out.append(int(torch.argmax(lg)))
        toks.append(out[-1])
    return out, margins


@pytest.mark.parametrize("graphs", [True, False])
@pytest.mark.parametrize("name,dtype", [("A", "float32"), ("A", "bfloat16"), ("B", "bfloat16"), ("C", "float32"), ("E", "bfloat16")])
def test_greedy_generation_through_the_entry_point(name, dtype, graphs, dirs):
    from lastengine_b200 import Engine, SamplingParams
    bf16 = dtype == "bfloat16"
    eng = Engine.from_pretrained(dirs[name], dtype=dtype, max_tokens=1024, use_graphs=graphs)
    prompts = reqs_for(name, [5, 1, 23, 66], 43)
    steps = 10
    res = eng.generate(prompts, SamplingParams(temperature=0.0), max_new_tokens=steps, stop_token_ids=[])
    compared = 0
    for p, got in zip(prompts, res.tokens):
        want, margins = plain_greedy(name, dirs, p, steps, bf16)
        assert len(got) == steps
        for i in range(steps):
            if margins[i] < 2 * TOL[dtype]:
                break
            assert got[i] == want[i], f"{name} {dtype}: prompt of {len(p)}, token {i}"
            compared += 1
    assert compared >= steps * len(prompts) // 3
    assert eng.cache.slots.n_held == 0
    eng.cache.check()


@pytest.mark.parametrize("name,dtype", [("A", "float32"), ("B", "bfloat16")])
def test_a_sequence_written_out_and_read_back_goes_on_where_it_stood(name, dtype, dirs):
    from lastengine_b200 import Engine
    eng = Engine.from_pretrained(dirs[name], dtype=dtype, max_tokens=512, max_seqs=4)
    r = reqs_for(name, [90], 44)[0]
    s = eng.new_sequence()
    eng.step([s], [r[:70]], None)
    data = eng.export_sequence(s)
    a = H.to_host(eng.step([s], [r[70:]], [list(range(20))]))
    other = eng.new_sequence()
    eng.step([other], [r[:5]], None)
    t = eng.import_sequence(data)
    assert t != s and eng.length(t) == 70
    b = H.to_host(eng.step([t], [r[70:]], [list(range(20))]))
    eng.release([s, other, t])
    assert H.rel_err(b, a) < 1e-6
    eng.cache.check()


def test_replay_program(dirs, tmp_path):
    """bin/trace_run on a folder of this design: three unequal requests start together, go on token by
    token and leave one by one."""
    import json
    import subprocess
    import sys
    name = "A"
    reqs = dict(zip("xyz", reqs_for(name, [12, 75, 3], 45)))
    first = {"x": 9, "y": 70, "z": 1}
    steps = [{"step": 0, "entries": [{"id": r, "tokens": reqs[r][:first[r]], "want": list(range(first[r]))} for r in "xyz"],
              "end": []}]
    fed, live, n = dict(first), ["x", "y", "z"], 1
    while live:
        ent = [{"id": r, "tokens": [reqs[r][fed[r]]], "want": [0]} for r in live]
        for r in live:
            fed[r] += 1
        ended = [r for r in live if fed[r] >= len(reqs[r])]
        steps.append({"step": n, "entries": ent, "end": ended})
        live = [r for r in live if r not in ended]
        n += 1
    out = str(tmp_path / "out")
    p = subprocess.run([sys.executable, os.path.join(H.ROOT, "bin", "trace_run"), "--model", dirs[name], "--dtype", "float32",
                        "--out", out, "--max-tokens", str(sum(len(t) for t in reqs.values()))],
                       input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True, timeout=900)
    assert p.returncode == 0, p.stderr[-2000:]
    assert [l for l in p.stdout.splitlines() if l.startswith("done")] == [f"done {i}" for i in range(n)]
    V = ALL[name]["vocab"]
    got = {r: [] for r in reqs}
    for st in steps:
        lg = torch.from_numpy(np.fromfile(os.path.join(out, f"{st['step']}.f32"), dtype="<f4").reshape(-1, V))
        at = 0
        for e in st["entries"]:
            got[e["id"]].append(lg[at:at + len(e["want"])])
            at += len(e["want"])
        assert at == lg.shape[0]
    for r, t in reqs.items():
        want, ok = plain(name, dirs, t, False)
        assert H.rel_err(torch.cat(got[r])[ok], want[ok]) < H.TOL_F32, r


def test_command_line_generates_samples_and_compares_the_two_number_formats(dirs):
    """bin/lastengine on a folder of this design: greedy and sampled generation (the same seed gives the same
    tokens), the dump of a greedy run, and bfloat16 against the 32-bit path step by step."""
    import json
    import subprocess
    import sys
    exe = os.path.join(H.ROOT, "bin", "lastengine")
    d = dirs["A"]
    base = [sys.executable, exe, "generate", "--model", d, "--prompt-ids", "1,2,3", "--prompt-ids", "9 8 7 6 5", "--max-new-tokens", "6",
            "--stop-token-id", "199"]
    p = subprocess.run(base + ["--dtype", "float32", "--temperature", "0"], capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-1500:]
    rows = [json.loads(l) for l in p.stdout.splitlines()]
    assert len(rows) == 2 and all(1 <= len(r["tokens"]) <= 6 for r in rows)
    want = plain_greedy("A", dirs, [1, 2, 3], 1, False)[0]
    assert rows[0]["tokens"][0] == want[0]
    sampled = [subprocess.run(base + ["--temperature", "0.9", "--top-k", "20", "--seed", "5"], capture_output=True, text=True, timeout=600)
               for _ in range(2)]
    assert sampled[0].returncode == 0 and sampled[0].stdout == sampled[1].stdout
    p2 = subprocess.run([sys.executable, exe, "tf-dump", d, "1,2,3", "6", "--dtype", "float32"], capture_output=True, text=True, timeout=600)
    assert p2.returncode == 0, p2.stderr[-1500:]
    dump = json.loads(p2.stdout.splitlines()[-1])
    if len(rows[0]["tokens"]) == 6:
        assert dump["gen_ids"] == rows[0]["tokens"]
    p3 = subprocess.run([sys.executable, exe, "dense-cmp", d, "1,2,3", "6"], capture_output=True, text=True, timeout=600)
    assert p3.returncode == 0, p3.stderr[-1500:]
    assert "/6 argmax agree, mean |dlogprob|" in p3.stdout.splitlines()[-1]
