"""The Zekivik configuration, plan and tensor list, and the plain implementation's own pieces (no GPU)."""
import copy
import os

import pytest
import torch

import plain_zekivik as P
from zekivik_configs import ALL, Z_A, Z_C, Z_D


def plan_of(cfg):
    from lastengine_b200.registry import plan_from_config
    return plan_from_config(cfg)


def test_runs_follow_the_loop():
    from lastengine_b200.config import ZekivikConfig
    assert ZekivikConfig.from_dict(Z_A).runs() == [(0, None), (1, 0), (2, None), (1, 1), (2, None), (3, None)]
    assert ZekivikConfig.from_dict(Z_C).runs() == [(0, 0), (1, None), (0, 1), (1, None), (0, 2), (1, None)]
    assert ZekivikConfig.from_dict(Z_D).runs() == [(0, None), (1, 0), (2, None)]
    for cfg in ALL.values():
        assert ZekivikConfig.from_dict(cfg).runs() == P.schedule(cfg)
    none = {k: v for k, v in Z_A.items() if k != "loop"}
    assert ZekivikConfig.from_dict(none).runs() == [(i, None) for i in range(4)]


def test_plan_schedule_cache_entries_and_stream_additions():
    plan = plan_of(Z_A)
    assert [e.layer for e in plan.schedule] == [0, 1, 2, 1, 2, 3]
    adds = {(a.before, a.embedding, a.row) for a in plan.stream_adds}
    assert adds == {(1, False, 0), (3, True, 1)}
    assert plan.stream_tables == {"loop.step": (2, 64)}
    from lastengine_b200.engine.model import Model
    from lastengine_b200.parts.base import BuildEnv, KVSpec, StateSpec
    m = Model(plan, BuildEnv(device=torch.device("cpu"), dtype=torch.float32))
    specs = m.cache_specs()
    assert len(specs) == 6                                   # every run of a layer has its own entry
    assert specs[0] == StateSpec((2, 16, 24), torch.float32)
    # key heads of 32 and value heads of 16 are cached 32 wide (a size the tensor-core kernels take); 16 and 48 stay
    assert specs[1] == specs[3] == (KVSpec(2, 32, 0, None), StateSpec((4 * 32 + 2 * 32 + 2 * 16, 2), torch.float32))
    assert specs[5][0] == KVSpec(1, 16, 0, 48)
    names = set(m.tensor_specs())
    assert {"embed.weight", "head.weight", "final.norm.weight", "loop.step", "l0.norm1.weight", "l0.norm2.weight",
            "l0.rg1", "l0.rg1.b", "l0.rg2", "l0.rg2.b", "l0.mix.q", "l0.mix.g", "l0.mlp.gate", "l1.mix.q.conv",
            "l3.mix.v.conv", "l3.mlp.down"} <= names
    assert not any(n.startswith(("l1.norm2", "l1.rg2", "l1.mlp", "l2.mlp")) for n in names)
    assert m.tensor_specs()["l1.mix.v.conv"].shape == (2 * 16, 3)
    assert m.tensor_specs()["l3.mix.o"].shape == (64, 2 * 48)
    # checkpoint spelling: the bare names
    assert plan.checkpoint_names("l0.norm1.weight") == "l0.norm1" and plan.tensor_aliases("l0.norm1") == "l0.norm1.weight"
    assert plan.checkpoint_names("l0.mix.q") == "l0.mix.q" and plan.tensor_aliases("head") == "head.weight"


def test_a_single_tap_keeps_no_state():
    from lastengine_b200.engine.model import Model
    from lastengine_b200.parts.base import BuildEnv, KVSpec
    m = Model(plan_of(Z_C), BuildEnv(device=torch.device("cpu"), dtype=torch.float32))
    assert m.cache_specs()[0] == KVSpec(1, 128, 0, None)


@pytest.mark.parametrize("edit,needle", [
    (lambda c: c.pop("width"), "width"),
    (lambda c: c["layers"][0].__setitem__("type", "mamba"), "unknown layer type"),
    (lambda c: c["layers"][1]["mixer"].pop("scale"), "scale"),
    (lambda c: c["layers"][1]["mixer"].__setitem__("kv_heads", 3), "do not divide"),
    (lambda c: c["layers"][0]["mixer"].__setitem__("decay", [0.5]), "decay"),
    (lambda c: c["layers"][0]["mixer"]["rot"].__setitem__("dims", 7), "even"),
    (lambda c: c["layers"][0]["mixer"]["rot"].__setitem__("dims", 32), "more than dim"),
    (lambda c: c["layers"][0]["mlp"].__setitem__("kind", "experts"), "unknown mlp kind"),
    (lambda c: c["loop"].__setitem__("stop", 9), "does not fit"),
    (lambda c: c.__setitem__("norm", 1e-5), "must be an object"),
])
def test_config_errors_name_the_key(edit, needle):
    from lastengine_b200.config import ConfigError
    cfg = copy.deepcopy(Z_A)
    edit(cfg)
    with pytest.raises(ConfigError, match=needle):
        plan_of(cfg)


def test_written_folder_reads_back_and_the_loader_names_what_is_wrong(tmp_path):
    from lastengine_b200.weights import write_model_dir
    from lastengine_b200.weights.safetensors_io import SafetensorsFile
    d = write_model_dir(Z_D, str(tmp_path / "m"), seed=3, norm_init="random")
    sf = SafetensorsFile(os.path.join(d, "model.safetensors"))
    names = set(sf.names())
    assert {"embed", "head", "final.norm", "loop.step", "l0.norm1", "l1.mix.q.conv", "l1.rg2.b"} <= names
    t = P.read_safetensors(os.path.join(d, "model.safetensors"))
    assert t["loop.step"].shape == (1, 40) and t["l1.mix.k.conv"].shape == (5 * 24, 4)
    lg = P.forward(Z_D, t, [1, 2, 3, 4, 5])
    assert lg.shape == (5, 97) and torch.isfinite(lg).all()


# ---- the plain implementation's mechanisms against closed forms ------------------------------------
def test_plain_retention_scan_is_the_decayed_sum():
    torch.manual_seed(0)
    T, H, d, e = 9, 2, 4, 3
    q, k, v = torch.randn(T, H, d).double(), torch.randn(T, H, d).double(), torch.randn(T, H, e).double()
    decay = torch.tensor([0.5, 1.0]).double()
    o = P.retention_scan(q, k, v, decay)
    for t in (0, 4, 8):
        for h in range(H):
            want = sum(decay[h] ** (t - j) * (q[t, h] @ k[j, h]) * v[j, h] for j in range(t + 1))
            assert torch.allclose(o[t, h], want, atol=1e-12)


def test_plain_conv_sees_zeros_before_the_start_and_nothing_ahead():
    u = torch.arange(1.0, 7.0).double()[:, None].repeat(1, 2)
    w = torch.tensor([[1.0, 10.0, 100.0], [0.0, 0.0, 1.0]]).double()
    y = P.causal_conv(u, w)
    assert y[:, 0].tolist() == [100.0, 210.0, 321.0, 432.0, 543.0, 654.0]      # w[:, taps-1] meets the current row
    assert y[:, 1].tolist() == u[:, 1].tolist()


def test_plain_rotation_keeps_norms_and_depends_on_distance_only():
    torch.manual_seed(1)
    a, b = torch.randn(1, 1, 12).double(), torch.randn(1, 1, 12).double()
    ra = P.rotate(a.repeat(3, 1, 1), torch.tensor([5, 105, 7]), 8, 100.0)
    rb = P.rotate(b.repeat(3, 1, 1), torch.tensor([2, 102, 7]), 8, 100.0)
    assert torch.allclose(ra.norm(dim=-1), a.norm(dim=-1).expand(3, 1))
    assert torch.equal(ra[..., 8:], a.repeat(3, 1, 1)[..., 8:])                  # the rest of the head passes unchanged
    assert torch.allclose((ra[0] * rb[0]).sum(), (ra[1] * rb[1]).sum(), atol=1e-9)
    assert torch.allclose(ra[2], P.rotate(a, torch.tensor([7]), 8, 100.0)[0])


def test_command_line_writes_and_describes_a_folder(tmp_path, capsys):
    import json
    from lastengine_b200.cli import main
    cfg = tmp_path / "c.json"
    cfg.write_text(json.dumps(Z_A))
    out = tmp_path / "model"
    assert main(["init", "--config", str(cfg), "--seed", "5", "--out", str(out)]) == 0
    capsys.readouterr()
    assert main(["inspect", str(out)]) == 0
    text = capsys.readouterr().out
    assert "architecture Zekivik: 4 layers, hidden 64, vocab 200" in text
    assert "layer 0: retention + gated_dense" in text and "layer 1: attention + no feed-forward" in text
    assert "layers run in the order 0 1 2 1 2 3" in text


def test_a_loop_over_no_layers_is_no_loop_and_its_table_is_passed_by(tmp_path):
    import json
    from lastengine_b200.weights import write_model_dir
    from lastengine_b200.weights.loader import check_names
    from lastengine_b200.engine.model import Model
    from lastengine_b200.parts.base import BuildEnv
    cfg = copy.deepcopy(Z_D)
    cfg["loop"] = {"start": 2, "stop": 2, "times": 3}
    plan = plan_of(cfg)
    assert [e.layer for e in plan.schedule] == [0, 1, 2] and not plan.stream_adds
    assert "loop.step" in plan.unused_tensors
    m = Model(plan, BuildEnv(device=torch.device("cpu"), dtype=torch.float32))
    assert "loop.step" not in m.tensor_specs()
