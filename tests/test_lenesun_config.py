"""The Lenesun configuration and plan, on the CPU: typed reading, errors that name the key, the
schedule's cache entries, tensor names and shapes, and a written folder read back."""
import copy
import os

import pytest
import torch

from lenesun_configs import ALL, L_A, L_C


def plan_of(cfg):
    from lastengine_b200.registry import plan_from_config
    return plan_from_config(cfg)


def test_every_size_and_constant_comes_from_the_file():
    from lastengine_b200.config.lenesun import LenesunConfig
    c = LenesunConfig.from_dict(L_A)
    assert (c.vocab, c.width, c.eps, c.residual_mult, c.embedding_scale) == (200, 64, 1e-6, 0.7, 2.0)
    m = c.layers[3].mixer
    assert (m.heads, m.dim, m.rot_dim, m.vdim, m.q_rank, m.kv_rank, m.scale, m.kv_from) == (2, 24, 16, 32, 8, 48, 0.25, 2)
    assert (m.rot.dims, m.rot.base) == (16, 500.0)
    assert c.layers[1].mlp is None
    f = c.layers[3].mlp
    assert (f.experts, f.top, f.ff, f.limit) == (5, 3, 16, 0.5)


@pytest.mark.parametrize("path,value,word", [
    (("width",), None, "width"),
    (("norm",), None, "norm"),
    (("embedding", "scale"), None, "scale"),
    (("residual_mult",), "x", "residual_mult"),
    (("layers", 0, "mixer", "kv_rank"), None, "kv_rank"),
    (("layers", 0, "mixer", "rot", "dims"), 7, "even"),
    (("layers", 0, "mixer", "rot", "dims"), 10, "rot_dim"),
    (("layers", 0, "type"), "attention", "unknown layer type"),
    (("layers", 0, "mlp", "kind"), "dense", "unknown mlp kind"),
    (("layers", 0, "mlp", "router", "top"), 9, "top"),
    (("layers", 0, "mlp", "expert", "limit"), 0.0, "limit"),
    (("layers", 1, "mixer", "kv_from"), 1, "earlier"),
    (("layers", 3, "mixer", "kv_from"), 1, "caches nothing"),
    (("layers", 3, "mixer", "kv_from"), 0, "must equal"),
])
def test_errors_name_the_key(path, value, word):
    from lastengine_b200.config.base import ConfigError
    cfg = copy.deepcopy(L_A)
    at = cfg
    for k in path[:-1]:
        at = at[k]
    if value is None:
        del at[path[-1]]
    else:
        at[path[-1]] = value
    with pytest.raises(ConfigError) as e:
        plan_of(cfg)
    assert word in str(e.value)


def test_plan_schedule_parts_and_cache_entries():
    from lastengine_b200.engine.model import Model
    from lastengine_b200.parts.base import BuildEnv, LatentSpec
    plan = plan_of(L_A)
    assert [(e.layer, e.cache, e.writes_cache) for e in plan.schedule] == \
        [(0, None, True), (1, 0, False), (2, None, True), (3, 2, False)]
    assert all(ls.block == "parallel_residual" and ls.block_params == {"mult": 0.7} for ls in plan.layers)
    assert plan.layers[1].ffn is None and plan.layers[0].ffn.kind == "topk_moe"
    assert plan.embedding.params["scale"] == 2.0 and plan.head.params["tied"]
    model = Model(plan, BuildEnv(device=torch.device("cpu"), dtype=torch.float32))
    assert model.cache_specs() == {0: LatentSpec(32, 8), 2: LatentSpec(48, 16)}
    specs = model.tensor_specs()
    assert specs["l0.mix.dkv"].shape == (32 + 8, 64) and "l1.mix.dkv" not in specs and "l1.mix.dkv.norm" not in specs
    assert specs["l1.mix.uq"].shape == (3 * (8 + 8), 16) and specs["l1.mix.uk"].shape == (3 * 8, 32)
    assert specs["l3.mix.uv"].shape == (2 * 32, 48) and specs["l3.mix.sink"].shape == (2,)
    assert specs["l3.mlp.e4.down"].shape == (64, 16) and specs["l3.mlp.router.b"].shape == (5,)
    assert "l1.mlp.router" not in specs and "head.weight" not in specs
    assert plan.tensor_aliases("l2.norm1") == "l2.norm1.weight" and plan.checkpoint_names("final.norm.weight") == "final.norm"


@pytest.mark.parametrize("name", list(ALL))
def test_a_written_folder_holds_the_designs_names_and_reads_back(name, tmp_path):
    from lastengine_b200.engine.model import Model
    from lastengine_b200.parts.base import BuildEnv
    from lastengine_b200.weights import write_model_dir
    from lastengine_b200.weights.safetensors_io import SafetensorsFile
    cfg = ALL[name]
    d = write_model_dir(cfg, str(tmp_path / name), seed=3)
    names = set(SafetensorsFile(os.path.join(d, "model.safetensors")).names())
    assert {"embed", "final.norm", "l0.norm1", "l0.mix.dq", "l0.mix.dq.norm", "l0.mix.sink", "l0.mix.o"} <= names
    assert not any(n.endswith(".weight") for n in names)
    plan = plan_of(cfg)
    model = Model(plan, BuildEnv(device=torch.device("cpu"), dtype=torch.float32))
    assert {plan.tensor_aliases(n) for n in names} == set(model.tensor_specs())


def test_latent_rows_are_paged_like_keys_and_go_out_and_come_back():
    """The cache's bookkeeping for latent rows on the CPU: pages per sequence, reuse, export and import."""
    from lastengine_b200.cache import Cache
    from lastengine_b200.parts.base import LatentSpec
    c = Cache({0: LatentSpec(28, 6), 2: LatentSpec(22, 10)}, max_tokens=256, max_seqs=3, dtype=torch.float32, device="cpu")
    assert len(c.kv_groups) == 2 and c.kv_groups[0].k_pool.shape == (1, 4, 1, 64, 34) and c.kv_groups[0].v_pool.numel() == 0
    a, b = c.alloc_seq(), c.alloc_seq()
    c.reserve({a: 70, b: 3})
    c.commit({a: 70, b: 3})
    g = c.kv_groups[0]
    pages = g.seq_pages[a]
    assert len(pages) == 2 and len(g.seq_pages[b]) == 1
    g.k_pool[0, pages[0], 0] = torch.arange(64 * 34, dtype=torch.float32).view(64, 34)
    g.k_pool[0, pages[1], 0, :6] = -1.0
    data = c.export_seq(a)
    assert len(data) == 8 + 70 * (34 + 32) * 4
    c.free_seq(a)
    d = c.alloc_seq()                 # takes the slot and, below, the pages that were just given back
    c.reserve({d: 5})
    c.commit({d: 5})
    e = c.import_seq(data)
    assert c.length(e) == 70
    pe = g.seq_pages[e]
    assert torch.equal(g.k_pool[0, pe[0], 0], torch.arange(64 * 34, dtype=torch.float32).view(64, 34))
    assert torch.equal(g.k_pool[0, pe[1], 0, :6], torch.full((6, 34), -1.0))
    c.check()
    with pytest.raises(Exception):
        c.reserve({e: 1000})
    c.check()


def test_inspect_prints_the_layers(tmp_path, capsys):
    from lastengine_b200.cli import main
    from lastengine_b200.weights import write_model_dir
    d = write_model_dir(L_C, str(tmp_path / "m"), seed=1)
    assert main(["inspect", d]) == 0
    out = capsys.readouterr().out
    assert "latent_attention" in out and "Lenesun" in out
