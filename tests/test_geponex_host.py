"""Geponex on the CPU: the configuration, the model's structure, the plain functions among themselves, and the
engine's host side (cache slots of layers that share weights, rows of state and of the shifted token, batching, scheduler)
over the torch stand-ins of the kernels."""
import copy
import math

import pytest
import torch

import helpers
import geponex_cases as cases
from plain import geponex_plain as plain


@pytest.fixture(scope="module")
def geponex_folders(tmp_path_factory):
    made = {}

    def get(name):
        if name not in made:
            made[name] = cases.make_folder(name, str(tmp_path_factory.mktemp(f"geponex_{name}")))
        return made[name]
    return get


def test_configuration_reads_every_size_and_round_trips():
    from vt_transformer_b200.config import ConfigError, config_from_dict
    from vt_transformer_b200.config.geponex import GeponexConfig
    cfg = config_from_dict(copy.deepcopy(cases.CONFIGS["mix"]))
    assert isinstance(cfg, GeponexConfig) and cfg.vocab == 300 and cfg.width == 64 and len(cfg.layers) == 6
    assert (cfg.norm_groups, cfg.postln_alpha, cfg.norm_eps) == (4, 2.5, 1e-5)
    att = cfg.layers[1].mixer
    assert (att.heads, att.dim, att.rot_dim, att.vdim, att.q_rank, att.kv_rank, att.scale, att.second) == (3, 24, 16, 40, 40, 48, 0.2, False)
    assert (att.rot.dims, att.rot.base) == (16, 3000.0)
    assert (att.rot.scaling.factor, att.rot.scaling.original, att.rot.scaling.fast, att.rot.scaling.slow) == (8.0, 64, 4.0, 1.0)
    assert cfg.layers[2].mixer.second and cfg.layers[2].mixer.rot.scaling is None and cfg.layers[2].mlp is None
    assert cfg.layers[0].mixer.decay == (0.7, 0.95, 1.0) and cfg.layers[1].mlp.ff == 100
    f = cfg.layers[0].mlp
    assert (f.experts, f.top, f.scale, f.ff, f.limit, f.shared_ff, f.shared_limit) == (5, 2, 2.0, 20, 1.5, 36, 3.0)
    assert cfg.layers[5].mlp.shared_ff is None
    assert [cfg.owner(i) for i in range(6)] == [0, 1, 2, 1, 0, 5]
    assert config_from_dict(cfg.to_dict()) == cfg
    one = copy.deepcopy(cases.CONFIGS["lightning_alone"])
    one["layers"][0]["mixer"]["decay"] = 0.9                       # one number stands for every head
    assert config_from_dict(one).layers[0].mixer.decay == (0.9, 0.9, 0.9)
    for spoil, match in ((lambda c: c["layers"][0].__setitem__("type", "other"), "layers\\[0\\].*'other'"),
                         (lambda c: c["layers"][1]["mixer"].pop("kv_rank"), "layers\\[1\\].mixer.*'kv_rank'"),
                         (lambda c: c["layers"][1]["mixer"]["rot"].__setitem__("dims", 18), "rot.dims"),
                         (lambda c: c["layers"][0]["mixer"].__setitem__("decay", [0.5]), "decay"),
                         (lambda c: c["layers"][0]["mlp"]["router"].__setitem__("top", 6), "top"),
                         (lambda c: c["layers"][3].__setitem__("weights_of", 9), "weights_of"),
                         (lambda c: c["layers"][3].__setitem__("weights_of", 2), "weights_of"),
                         (lambda c: c["norm"].__setitem__("groups", 5), "groups")):
        bad = copy.deepcopy(cases.CONFIGS["mix"])
        spoil(bad)
        with pytest.raises(ConfigError, match=match):
            config_from_dict(bad)


def test_a_layer_that_uses_anothers_weights_has_a_cache_and_a_shift_row_of_its_own():
    from vt_transformer_b200.config import config_from_dict, get_architecture
    from vt_transformer_b200.models.base import DecoderModel
    from vt_transformer_b200.parts import Runtime, StateSpec
    from vt_transformer_b200.parts.base import LatentCacheSpec
    cfg = config_from_dict(copy.deepcopy(cases.CONFIGS["mix"]))
    model = DecoderModel(get_architecture(cfg.architecture).model_spec(cfg), Runtime(torch.device("cpu"), torch.float32, None))
    assert [r.block for r in model.spec.order] == [0, 1, 2, 1, 0, 3]
    assert [r.cache for r in model.spec.order] == [(2 * i, 2 * i + 1) for i in range(6)]
    slots = model.cache_slots()
    assert sorted(slots) == list(range(12))
    assert all(isinstance(slots[2 * i], StateSpec) and slots[2 * i].shape == (64,) for i in range(6))      # the token before, a layer
    assert [type(slots[2 * i + 1]) for i in range(6)] == [StateSpec, LatentCacheSpec, LatentCacheSpec, LatentCacheSpec, StateSpec, LatentCacheSpec]
    assert slots[3] == slots[7] == LatentCacheSpec(48 + 16) and slots[1].shape == slots[9].shape == (3, 24, 40)
    names = set(model.param_specs())
    assert {"embed", "final.norm", "l0.norm1", "l0.norm2", "l0.shift", "l1.mix.dq.norm", "l1.mix.dkv", "l1.mix.uk", "l2.mix.sink", "l2.mix.g",
            "l0.mix.norm", "l0.mix.g", "l1.mlp.up.b", "l1.mlp.act", "l0.mlp.router", "l0.mlp.e4.down", "l0.mlp.shared.up", "l5.mlp.e5.gate"} <= names
    assert not any(n.startswith(("l3.", "l4.")) for n in names)
    assert "l2.norm2" not in names and "l1.mix.sink" not in names and "l1.mix.g" not in names and "l5.mlp.shared.up" not in names
    assert "head" not in names or model.param_specs()["head"].optional          # the output head is the embedding table
    assert model.graph_safe()


def test_ramped_frequencies_hit_every_branch():
    from vt_transformer_b200.parts.rope import ramped_frequencies
    for dims, base, sc in ((16, 3000.0, (8.0, 64, 4.0, 1.0)), (32, 5e4, (3.0, 40, 2.0, 0.5)), (8, 777.0, (6.0, 32, 8.0, 1.0)),
                           (32, 1e4, (4.0, 256, 16.0, 2.0))):
        want, m = plain.rotary_frequencies(dims, base, dict(zip(("factor", "original", "fast", "slow"), sc)))
        got, gm = ramped_frequencies(dims, base, sc)
        assert float((got.double() / want - 1).abs().max()) < 1e-6 and abs(gm - m) < 1e-12 and abs(m - (0.1 * math.log(sc[0]) + 1)) < 1e-12
        plainf = torch.tensor([base ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=torch.float64)
        ratio = want / plainf
        assert ratio[0] == 1.0 and abs(float(ratio[-1]) - 1 / sc[0]) < 1e-12
    # the 32-dimension cases have pairs before the ramp, on it and after it
    want, _ = plain.rotary_frequencies(32, 5e4, {"factor": 3.0, "original": 40, "fast": 2.0, "slow": 0.5})
    ratio = want / torch.tensor([5e4 ** (-2.0 * i / 32) for i in range(16)], dtype=torch.float64)
    assert int((ratio == 1).sum()) >= 1 and int(((ratio < 1) & (ratio > 1 / 3 + 1e-9)).sum()) >= 1 and int(((ratio - 1 / 3).abs() < 1e-12).sum()) >= 1


def test_plain_functions_agree_with_their_definitions():
    g = torch.Generator().manual_seed(3)
    v = torch.randn((5, 24), generator=g, dtype=torch.float64)
    w = torch.randn(24, generator=g, dtype=torch.float64)
    out = plain.grouped_rms_norm(v, w, 1e-5, 3)
    for t in range(5):
        for k in range(3):
            part = v[t, 8 * k:8 * k + 8]
            assert torch.allclose(out[t, 8 * k:8 * k + 8], part / math.sqrt(float((part * part).mean()) + 1e-5) * w[8 * k:8 * k + 8])
    assert torch.allclose(plain.grouped_rms_norm(v, w, 1e-5, 1), plain.rms_norm(v, w, 1e-5))
    mu = torch.rand(24, generator=g, dtype=torch.float64)
    before = torch.randn(24, generator=g, dtype=torch.float64)
    shifted, carry = plain.token_shift(v, before, mu)
    assert torch.allclose(shifted[0], v[0] + (before - v[0]) * mu) and torch.allclose(shifted[3], v[3] + (v[2] - v[3]) * mu)
    assert torch.equal(carry, v[4])
    # the softmax with a sink: the weights and the sink's share add up to one; without keys' scores the sink is not scaled
    q, k = torch.randn((1, 2, 4), generator=g, dtype=torch.float64), torch.randn((3, 2, 4), generator=g, dtype=torch.float64)
    ones = torch.ones((3, 2, 1), dtype=torch.float64)
    sink = torch.tensor([0.3, -1.0], dtype=torch.float64)
    total = plain.softmax_attention(q, k, ones, torch.tensor([2]), 0.5, sink)[0, :, 0]
    s = torch.einsum("hd,jhd->hj", q[0], k) * 0.5
    assert torch.allclose(total, torch.exp(s).sum(1) / (torch.exp(s).sum(1) + torch.exp(sink)))
    # xIELU is continuous at zero with slope 1/2 on both sides, and the expert's gate is clamped from above only
    p, qq = torch.tensor(0.4, dtype=torch.float64), torch.tensor(-0.2, dtype=torch.float64)
    z = torch.tensor([-1e-6, 0.0, 1e-6], dtype=torch.float64)
    assert torch.allclose(plain.xielu(z, p, qq), z / 2, atol=1e-10)
    h = torch.tensor([[1.0]], dtype=torch.float64)
    one = torch.tensor([[1.0]], dtype=torch.float64)
    assert float(plain.expert(h * -9, one, one * 0, one, 2.0)) == pytest.approx(-9 / (1 + math.exp(1.702 * 9)))
    assert float(plain.expert(h * 9, one, one, one, 2.0)) == pytest.approx(2 / (1 + math.exp(-1.702 * 2)) * 3.0)
    assert float(plain.expert(h * 9, one, -one, one, 2.0)) == pytest.approx(2 / (1 + math.exp(-1.702 * 2)) * -1.0)


@pytest.mark.parametrize("family", ["whole", "tail", "portions", "mixed"])
def test_cuts_equal_the_plain_implementation(fake_backend, geponex_folders, family):
    cases.replay(geponex_folders("mix"), cases.prompts_for("mix"), family, "cpu", "float32")


@pytest.mark.parametrize("name", ["wide", "latent_alone", "latent2_alone", "lightning_alone", "dense_alone", "experts_alone"])
def test_other_sizes_and_each_mechanism_alone(fake_backend, geponex_folders, name):
    prompts = cases.prompts_for(name, lengths=[1, 12, 45])
    for family in ("whole", "portions", "mixed"):
        cases.replay(geponex_folders(name), prompts, family, "cpu", "float32", alone=name.endswith("alone"))


def test_tokens_grouped_by_expert_equal_the_plain_implementation(fake_backend, geponex_folders, monkeypatch):
    from vt_transformer_b200 import ops
    monkeypatch.setattr(ops, "EXPERTS_GROUPED_MIN_PICKS", 1)
    for name in ("mix", "experts_alone"):
        cases.replay(geponex_folders(name), cases.prompts_for(name), "portions", "cpu", "float32")
        cases.replay(geponex_folders(name), cases.prompts_for(name), "mixed", "cpu", "float32")


def test_greedy_generation_through_the_entry_point(fake_backend, geponex_folders):
    cases.greedy_generation(geponex_folders("mix"), "mix", "cpu", "float32", n_new=6)


def test_a_tensor_of_the_wrong_shape_is_refused(fake_backend, geponex_folders, tmp_path):
    from vt_transformer_b200.weights import WeightError

    def spoil(t):
        t["l1.mix.uk"] = t["l1.mix.uk"][:-1]
    with pytest.raises(WeightError):
        cases.runner_for(cases.rewritten(geponex_folders("mix"), str(tmp_path / "bad"), spoil), "cpu", "float32", num_pages=4)


def test_random_weights_mode_of_the_command_line_writes_a_folder_that_loads(tmp_path):
    import json
    import os
    import subprocess
    import sys
    cfg = tmp_path / "cfg.json"
    cfg.write_text(json.dumps(cases.CONFIGS["mix"]))
    out = tmp_path / "model"
    res = subprocess.run([sys.executable, "-m", "vt_transformer_b200", "random-weights", "--config", str(cfg), "--out", str(out),
                          "--seed", "5", "--sigma", "0.05"], capture_output=True, text=True, timeout=600,
                         env=dict(os.environ, PYTHONPATH=helpers.ROOT), cwd=helpers.ROOT)
    assert res.returncode == 0, res.stderr
    from vt_transformer_b200.config import config_from_dict, load_config
    from vt_transformer_b200.weights import SafetensorsSource, check_against
    from vt_transformer_b200.weights.random_init import parameter_table
    config = load_config(str(out))
    assert config == config_from_dict(copy.deepcopy(cases.CONFIGS["mix"]))
    check_against(SafetensorsSource(str(out)), parameter_table(config))
