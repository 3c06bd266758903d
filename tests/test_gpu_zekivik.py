"""The Zekivik decoder on the GPU against the plain implementation (tests/plain_zekivik.py): every
mechanism alone, then whole models: prompts whole, in portions and token by token, unequal batches,
slots and pages used again, long decoding, and greedy generation through the entry point."""
import os

import numpy as np
import pytest
import torch

import harness as H
import plain_zekivik as P
from zekivik_configs import ALL, Z_A, Z_B, att, ret

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}
TOL = {"float32": H.TOL_F32, "bfloat16": H.TOL_BF16}


def K():
    from lastengine_b200.ops import kernels
    return kernels


# ---- a mixer alone: its own cache, steps laid out as the engine lays them out ----------------------
class MixerRig:
    def __init__(self, kind, params, dtype, seed=0, std=0.3, max_tokens=2048, max_seqs=6, edit=None):
        from lastengine_b200.cache import Cache
        from lastengine_b200.engine.batch import BatchBuilder
        from lastengine_b200.engine.workspace import Workspace
        from lastengine_b200.parts.base import BuildEnv
        from lastengine_b200.registry import MIXERS
        from lastengine_b200.weights.loader import kept_dtype
        from lastengine_b200.weights.random_init import random_tensor
        dev = torch.device(DEV)
        self.env = BuildEnv(device=dev, dtype=DT[dtype], workspace=Workspace(dev))
        self.mixer = MIXERS.get(kind)(**params)
        self.plain = {}
        tens = {}
        for name, spec in self.mixer.tensors().items():
            t = random_tensor(name, spec, seed, std).to(torch.bfloat16).float()
            self.plain[name] = t.double()
            tens[name] = t
        if edit:
            edit(self.plain)
            tens = {n: v.float() for n, v in self.plain.items()}
        self.mixer.load({n: v.to(dev, kept_dtype(self.mixer.tensors()[n], torch.bfloat16, DT[dtype]))
                         for n, v in tens.items()}, self.env)
        self.cache = Cache({0: self.mixer.cache_spec()}, max_tokens=max_tokens, max_seqs=max_seqs, dtype=DT[dtype], device=dev)
        self.builder = BatchBuilder(dev)
        self.D = params["hidden_size"]

    def step(self, slots, hs):
        """hs: per sequence a [n, D] double tensor of mixer inputs; returns the mixer's outputs per sequence."""
        grow = {s: h.shape[0] for s, h in zip(slots, hs)}
        pos0 = [self.cache.length(s) for s in slots]
        self.cache.reserve(grow)
        tables = {gi: g.table(list(slots), max(1, max(len(g.seq_pages.get(s, ())) for s in slots)))
                  for gi, g in enumerate(self.cache.kv_groups)}
        batch = self.builder.build(list(slots), [[0] * h.shape[0] for h in hs], pos0, [], tables)
        h = torch.cat(hs, 0).to(DEV, self.env.dtype)
        out = torch.zeros(h.shape[0], self.D, dtype=torch.float32, device=DEV)
        self.mixer.forward(h, out, False, batch, self.cache.view(0, True, batch.tables), self.env)
        K().check_device_status()
        self.cache.commit(grow)
        return list(torch.split(out.double().cpu(), [x.shape[0] for x in hs]))


def inputs(T, D, seed, bf16):
    g = torch.Generator().manual_seed(seed)
    h = torch.randn(T, D, generator=g, dtype=torch.float64)
    return P.round_bf16(h) if bf16 else h


RET_CASES = [  # heads, dim, vdim, decay, rot dims
    (2, 16, 24, [0.9, 0.99], 8),
    (1, 48, 16, [1.0], 48),
    (3, 32, 64, [0.5, 0.97, 0.0], 0),
    (2, 128, 128, [0.999, 0.98], 64),
    (1, 256, 96, [0.95], 32),
]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H_,d,e,decay,rot", RET_CASES)
def test_retention_alone_whole_in_portions_and_batched(H_, d, e, decay, rot, dtype):
    bf16 = dtype == "bfloat16"
    D = 40
    m = ret(H_, d, e, decay, rot, 777.0)
    pos = {"kind": "rope", "params": {"rope_dim": rot, "theta": 777.0}} if rot else None
    from lastengine_b200.parts.base import PartSpec
    params = dict(hidden_size=D, num_heads=H_, head_dim=d, v_head_dim=e, decay=decay, norm_eps=1e-5,
                  position=PartSpec(**pos) if pos else None, names=("q", "k", "v", "g", "o"))
    rig = MixerRig("retention", params, dtype, seed=5)
    rnd = P.round_bf16 if bf16 else P.identity
    hs = [inputs(n, D, 10 + n, bf16) for n in (150, 1, 37)]
    want = [P.retention_mixer(h, rig.plain, m, 1e-5, rnd) for h in hs]
    tol = TOL[dtype]
    # each alone, whole
    for h, w in zip(hs, want):
        s = rig.cache.alloc_seq()
        got = rig.step([s], [h])[0]
        rig.cache.free_seq(s)
        assert H.rel_err(got, w) < tol
    # together (unequal), then each goes on alone in portions of 2, 1, 5, ...
    more = [inputs(21, D, 50 + i, bf16) for i in range(3)]
    want2 = [P.retention_mixer(torch.cat([h, x]), rig.plain, m, 1e-5, rnd) for h, x in zip(hs, more)]
    slots = [rig.cache.alloc_seq() for _ in hs]          # the slots just freed: their state must start at zero
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


def test_retention_keeps_a_key_from_far_back():
    """A head that does not decay: a key written at position 2 is met by the query at position 600
    (scaled so that this one product stands out); a state that was lost, reset or decayed shows."""
    D, d, e = 32, 16, 16
    m = ret(2, d, e, [1.0, 0.9], 0, 1.0)
    params = dict(hidden_size=D, num_heads=2, head_dim=d, v_head_dim=e, decay=[1.0, 0.9], norm_eps=1e-6,
                  names=("q", "k", "v", "g", "o"))
    rig = MixerRig("retention", params, "float32", seed=8)
    h = inputs(601, D, 3, False) * 0.05
    h[2] = h[2] * 40
    h[600] = h[600] * 40
    want = P.retention_mixer(h, rig.plain, m, 1e-6)
    gone = P.retention_mixer(h[3:], rig.plain, m, 1e-6)
    assert H.rel_err(gone[-1:], want[-1:]) > 0.05            # the far key matters to the last row
    s = rig.cache.alloc_seq()
    a = rig.step([s], [h[:590]])[0]
    tail = torch.cat([rig.step([s], [h[i:i + 1]])[0] for i in range(590, 601)])
    assert H.rel_err(torch.cat([a, tail]), want) < H.TOL_F32
    assert H.rel_err(tail[-1:], want[-1:]) < H.TOL_F32


ATT_CASES = [  # heads, kv, dim, vdim, taps, scale, rot dims
    (4, 2, 32, 16, 3, 0.2, 16),
    (2, 1, 16, 48, 2, 0.3, 16),
    (3, 3, 64, 64, 5, 0.125, 64),
    (4, 1, 128, 128, 1, 0.09, 32),
    (5, 5, 24, 40, 4, 0.25, 0),
    (2, 2, 96, 32, 2, 0.1, 48),
    (6, 2, 64, 32, 3, 0.15, 64),       # cached 64 wide: the tensor-core kernels with zero-padded values
    (2, 2, 32, 128, 2, 0.2, 16),       # cached 128 wide: zero-padded queries and keys
]


def att_params(D, heads, kv, dim, vdim, taps, scale, rot, base=5000.0):
    from lastengine_b200.parts.base import PartSpec
    return dict(hidden_size=D, num_heads=heads, num_kv_heads=kv, head_dim=dim, v_head_dim=vdim, norm_eps=1e-5,
                qk_norm="unit", v_norm=True, conv_taps=taps, scale=scale, output_gate=True,
                position=PartSpec("rope", {"rope_dim": rot, "theta": base}) if rot else PartSpec("none"),
                names={"q": "q", "k": "k", "v": "v", "o": "o", "gate": "g", "q_conv": "q.conv", "k_conv": "k.conv",
                       "v_conv": "v.conv"})


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("heads,kv,dim,vdim,taps,scale,rot", ATT_CASES)
def test_attention_alone_whole_in_portions_and_batched(heads, kv, dim, vdim, taps, scale, rot, dtype):
    bf16 = dtype == "bfloat16"
    D = 48
    m = att(heads, kv, dim, vdim, taps, scale, rot, 5000.0)
    rig = MixerRig("attention", att_params(D, heads, kv, dim, vdim, taps, scale, rot), dtype, seed=6)
    rnd = P.round_bf16 if bf16 else P.identity
    tol = TOL[dtype]
    hs = [inputs(n, D, 20 + n, bf16) for n in (131, 2, 64)]      # over two page borders, two tokens, exactly a page
    want = [P.attention_mixer(h, rig.plain, m, 1e-5, rnd) for h in hs]
    for h, w in zip(hs, want):
        s = rig.cache.alloc_seq()
        assert H.rel_err(rig.step([s], [h])[0], w) < tol
        rig.cache.free_seq(s)
    more = [inputs(12, D, 70 + i, bf16) for i in range(3)]
    want2 = [P.attention_mixer(torch.cat([h, x]), rig.plain, m, 1e-5, rnd) for h, x in zip(hs, more)]
    slots = [rig.cache.alloc_seq() for _ in hs]          # slots and pages that were just given back
    for g, w in zip(rig.step(slots, hs), want):
        assert H.rel_err(g, w) < tol
    cuts = [0, 1, 3, 4, 10, 12]                          # portions of 1, 2, 1, 6, 2 rows: shorter than the taps too
    outs = [[] for _ in hs]
    for a, b in zip(cuts[:-1], cuts[1:]):
        for i, g in enumerate(rig.step(slots, [x[a:b] for x in more])):
            outs[i].append(g)
    for i, w in enumerate(want2):
        assert H.rel_err(torch.cat(outs[i]), w[hs[i].shape[0]:]) < tol, f"sequence {i} after portions"


@pytest.mark.parametrize("vdim", [32, 64])
def test_attention_reaches_a_key_far_back_and_at_page_borders(vdim):
    """Inputs and weights made so that the query at the last position meets one far key with a score
    far above the rest: an unrotated dimension of head 0 carries a large value at those two rows."""
    D, dim = 32, 64
    rot = 32

    def edit(t):
        for n in ("q", "k"):
            t[n][rot] = 0.0
            t[n][rot, 0] = 3.0                      # dimension `rot` of head 0 reads input channel 0
        for n in ("q.conv", "k.conv"):
            t[n][rot] = 0.0
            t[n][rot, -1] = 1.0                     # and passes the convolution unchanged

    for far in (3, 63, 64, 65, 127, 128, 500):
        rig = MixerRig("attention", att_params(D, 2, 1, dim, vdim, 3, 1.0, rot), "float32", seed=9, std=0.1, edit=edit)
        m = att(2, 1, dim, vdim, 3, 1.0, rot, 5000.0)
        T = 700
        h = inputs(T, D, 4, False) * 0.3
        h[:, 0] = 0.0
        h[far, 0] = 30.0
        h[T - 1, 0] = 30.0
        want = P.attention_mixer(h, rig.plain, m, 1e-5)
        cut = torch.cat([h[:far], h[far + 1:]])
        assert H.rel_err(P.attention_mixer(cut, rig.plain, m, 1e-5)[-1:], want[-1:]) > 0.02      # a thousand tolerances
        s = rig.cache.alloc_seq()
        whole = rig.step([s], [h])[0]
        rig.cache.free_seq(s)
        assert H.rel_err(whole, want) < H.TOL_F32
        s = rig.cache.alloc_seq()
        head = rig.step([s], [h[:T - 3]])[0]
        tail = torch.cat([rig.step([s], [h[i:i + 1]])[0] for i in range(T - 3, T)])
        assert H.rel_err(torch.cat([head, tail]), want) < H.TOL_F32, f"far key at {far}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("taps", [1, 2, 4, 7])
def test_causal_conv_kernel_and_its_state(taps, dtype):
    k = K()
    dt = DT[dtype]
    C = 200
    g = torch.Generator().manual_seed(taps)
    w = torch.randn(C, taps, generator=g)
    seqs = [torch.randn(n, C + 8, generator=g).to(dt) for n in (9, 1, 30)]       # the kernel reads a column slice
    want = [P.causal_conv(u[:, :C].double(), w.double()) for u in seqs]
    from lastengine_b200.engine.batch import BatchBuilder
    builder = BatchBuilder(torch.device(DEV))
    state = torch.zeros(4, C, max(taps - 1, 1), device=DEV)[:, :, : taps - 1].contiguous()
    state[3] = 7.0                                                               # a slot nobody uses stays as it is
    got = [[] for _ in seqs]
    fed = [0, 0, 0]
    for sizes in ([4, 1, 2], [1, None, 1], [2, None, 27], [2, None, None]):      # portions shorter than the taps too
        live = [i for i, n in enumerate(sizes) if n]
        u = torch.cat([seqs[i][fed[i]:fed[i] + sizes[i]] for i in live]).to(DEV)
        b = builder.build([i for i in live], [[0] * sizes[i] for i in live], [fed[i] for i in live], [], {})
        y = torch.zeros(u.shape[0], C, dtype=dt, device=DEV)
        k.causal_conv(y, u[:, :C], w.to(DEV), state if taps > 1 else None, b)
        r = 0
        for i in live:
            got[i].append(y[r:r + sizes[i]].double().cpu())
            r += sizes[i]
            fed[i] += sizes[i]
    for i, wnt in enumerate(want):
        assert H.rel_err(torch.cat(got[i]), wnt) < (1e-6 if dtype == "float32" else 8e-3)
    if taps > 1:
        assert torch.equal(state[3], torch.full_like(state[3], 7.0))
        assert torch.allclose(state[2].cpu().double(), seqs[2][30 - (taps - 1):, :C].double().T)


def test_small_kernels_gated_activation_gated_sum_and_stream_addition():
    k = K()
    g = torch.Generator().manual_seed(1)
    M, F, D = 37, 56, 40
    gu = torch.randn(M, 2 * F, generator=g) * 3
    out = torch.zeros(M, F, device=DEV)
    k.gated_act(out, gu.to(DEV), k.GELU_TANH)
    assert H.rel_err(out, P.gelu_tanh(gu[:, :F].double()) * gu[:, F:].double()) < 1e-6
    outb = torch.zeros(M, F, device=DEV, dtype=torch.bfloat16)
    k.gated_act(outb, gu.to(DEV), k.GELU_TANH)
    assert H.rel_err(outb, P.gelu_tanh(gu[:, :F].double()) * gu[:, F:].double()) < 5e-3
    x, y, z, b = torch.randn(M, D, generator=g), torch.randn(M, D, generator=g), torch.randn(M, D, generator=g) * 4, torch.randn(D, generator=g)
    xd = x.to(DEV)
    k.gated_residual(xd, y.to(DEV), z.to(DEV), b.to(DEV))
    assert H.rel_err(xd, x.double() + y.double() * P.sigmoid(z.double() + b.double())) < 1e-6
    x0, vec = torch.randn(M, D, generator=g), torch.randn(D, generator=g)
    xd = x.to(DEV)
    k.stream_add(xd, x0.to(DEV), vec.to(DEV))
    k.stream_add(xd, None, vec.to(DEV))
    assert H.rel_err(xd, x.double() + x0.double() + 2 * vec.double()) < 1e-6


@pytest.mark.parametrize("M,Kd,F", [(1, 64, 48), (8, 96, 160), (16, 256, 512), (40, 128, 256), (128, 256, 2048),
                                   (300, 64, 96), (700, 512, 1024), (1100, 256, 4096)])
def test_gated_gelu_as_the_epilogue_of_every_bfloat16_product(M, Kd, F):
    """Rows from one to over a thousand reach the weight stream, the sliced and the tiled tensor-core
    products and the one on pairs of SMs; each applies gelu(gate) * up before it stores."""
    from lastengine_b200.parts.ffn import fuse_gate_up
    k = Kd
    g = torch.Generator().manual_seed(M)
    x = P.round_bf16(torch.randn(M, k, generator=g, dtype=torch.float64))
    wg = P.round_bf16(torch.randn(F, k, generator=g, dtype=torch.float64) * (2.0 / k ** 0.5))
    wu = P.round_bf16(torch.randn(F, k, generator=g, dtype=torch.float64) / k ** 0.5)
    want = P.gelu_tanh(x @ wg.T) * (x @ wu.T)
    w = fuse_gate_up(wg.to(DEV, torch.bfloat16), wu.to(DEV, torch.bfloat16), True)
    for dt, tol in ((torch.bfloat16, 8e-3), (torch.float32, 2e-4)):
        out = torch.zeros(M, F, dtype=dt, device=DEV)
        K().linear(out, x.to(DEV, torch.bfloat16), w, K().GEGLU)
        K().check_device_status()
        assert H.rel_err(out, want) < tol
    silu = torch.zeros(M, F, dtype=torch.float32, device=DEV)          # the other activation is still what it was
    K().linear(silu, x.to(DEV, torch.bfloat16), w, K().SWIGLU)
    assert H.rel_err(silu, P.silu(x @ wg.T) * (x @ wu.T)) < 2e-4


# ---- whole models --------------------------------------------------------------------------------
@pytest.fixture(scope="module")
def dirs(tmp_path_factory):
    from lastengine_b200.weights import write_model_dir
    return {n: write_model_dir(cfg, str(tmp_path_factory.mktemp("z" + n)), seed=11 + i, norm_init="random")
            for i, (n, cfg) in enumerate(ALL.items())}


_plain = {}


def plain(name, dirs, tokens, bf16):
    key = (name, tuple(tokens), bf16)
    if key not in _plain:
        t = P.read_safetensors(os.path.join(dirs[name], "model.safetensors"))
        _plain[key] = P.forward(ALL[name], t, tokens, rnd=P.round_bf16 if bf16 else P.identity)
    return _plain[key]


def close(got, want, dtype) -> bool:
    """32-bit: every position within the tolerance.  bfloat16: a retention head's result is divided by
    its root mean square and the attention's queries and keys by theirs, so a position where those are
    small amplifies rounding noise tenfold (the plain implementation in bfloat16 is up to 2.7e-2 from
    itself in 32-bit at single positions of these models, at a median of 2e-3 to 4e-3); two bfloat16
    computations that round at different places can therefore be compared over the positions, not at
    each: half of them within a third of the tolerance and nine in ten within it.  What a single
    position must hold is tested in 32-bit, and in bfloat16 on each mixer alone."""
    if dtype == "float32":
        return H.rel_err(got, want) < H.TOL_F32
    want = want.double()
    e = (got.double().cpu() - want).abs().amax(dim=-1) / want.abs().max()
    if e.numel() < 8:
        return bool(e.max() < 3 * H.TOL_BF16)
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
    # a prompt in portions of several sizes, down to two tokens and one
    s = eng.new_sequence()
    outs, at = [], 0
    for n in (2, 1, 2, 59, 1, 64, 3, 18):
        outs.append(H.to_host(eng.step([s], [reqs[0][at:at + n]], [list(range(n))], check=True)))
        at += n
    eng.release(s)
    assert at == 150 and close(torch.cat(outs), want[0], dtype)
    # unequal requests in one batch (prompts of different lengths, then token by token, leaving one by one)
    got = H.run_batch(eng, reqs, [100, 1, 64, 1])
    for g, w, r in zip(got, want, reqs):
        assert close(g, w, dtype), f"batched, {len(r)} tokens"
    # the same again in the slots and pages that were just given back, in another order
    got = H.run_batch(eng, reqs[::-1], [1, 7, 2, 149])
    for g, w in zip(got, want[::-1]):
        assert close(g, w, dtype)
    assert eng.cache.slots.n_held == 0
    eng.cache.check()


@pytest.mark.parametrize("name", ["A", "D"])
def test_logits_do_not_depend_on_the_cut_or_the_batch_beyond_rounding(name, dirs):
    """32-bit: a position's logits whole, in portions, decoded and beside other requests agree far
    inside the tolerance against the plain implementation."""
    from lastengine_b200 import Engine
    eng = Engine.from_pretrained(dirs[name], dtype="float32", max_tokens=1024, max_seqs=6)
    reqs = reqs_for(name, [140, 9], 41)
    whole = H.run_whole(eng, reqs[0])
    tail = H.run_tail(eng, reqs[0], tail=80)
    batched = H.run_batch(eng, reqs, [61, 4])[0]
    assert H.rel_err(tail, whole) < 5e-6 and H.rel_err(batched, whole) < 5e-6


@pytest.mark.parametrize("name,dtype", [("A", "float32"), ("C", "float32"), ("B", "bfloat16")])
def test_long_decoding_from_a_short_prompt(name, dtype, dirs):
    from lastengine_b200 import Engine
    eng = Engine.from_pretrained(dirs[name], dtype=dtype, max_tokens=512, max_seqs=2)
    r = reqs_for(name, [200], 42)[0]
    got = H.run_tail(eng, r, tail=196)
    assert close(got, plain(name, dirs, r, dtype == "bfloat16"), dtype)


def plain_greedy(name, dirs, prompt, n, bf16):
    toks, out, margins = list(prompt), [], []
    for _ in range(n):
        lg = plain(name, dirs, toks, bf16)[-1]
        top = torch.topk(lg, 2).values
        margins.append(float((top[0] - top[1]) / lg.abs().max()))
        out.append(int(torch.argmax(lg)))
        toks.append(out[-1])
    return out, margins


@pytest.mark.parametrize("graphs", [True, False])
@pytest.mark.parametrize("name,dtype", [("A", "float32"), ("A", "bfloat16"), ("B", "bfloat16"), ("C", "float32"), ("D", "float32")])
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
            if margins[i] < TOL[dtype]:
                break
            assert got[i] == want[i], f"{name} {dtype}: prompt of {len(p)}, token {i}"
            compared += 1
    assert compared >= steps * len(prompts) // 3
    assert eng.cache.slots.n_held == 0
    eng.cache.check()


@pytest.mark.parametrize("name,dtype", [("A", "float32"), ("B", "bfloat16")])
def test_a_sequence_written_out_and_read_back_goes_on_where_it_stood(name, dtype, dirs):
    """Keys, values, the convolution's memory and the retention state of every layer run go out as bytes
    and come back into other slots and pages."""
    from lastengine_b200 import Engine
    eng = Engine.from_pretrained(dirs[name], dtype=dtype, max_tokens=512, max_seqs=4)
    r = reqs_for(name, [90], 44)[0]
    s = eng.new_sequence()
    eng.step([s], [r[:70]], None)
    data = eng.export_sequence(s)
    a = H.to_host(eng.step([s], [r[70:]], [list(range(20))]))
    other = eng.new_sequence()                       # the copy lands in another slot and other pages
    eng.step([other], [r[:5]], None)
    t = eng.import_sequence(data)
    assert t != s and eng.length(t) == 70
    b = H.to_host(eng.step([t], [r[70:]], [list(range(20))]))
    eng.release([s, other, t])
    assert H.rel_err(b, a) < 1e-6
    eng.cache.check()


def test_replay_program_with_a_cache_sized_to_the_tokens_alone(dirs, tmp_path):
    """bin/trace_run with --max-tokens equal to the tokens the live requests hold, not rounded up to pages:
    three unequal requests start together (the shortest with one token), go on token by token and leave one
    by one; every request's last page is partly filled."""
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
        assert H.rel_err(torch.cat(got[r]), plain(name, dirs, t, False)) < H.TOL_F32, r
