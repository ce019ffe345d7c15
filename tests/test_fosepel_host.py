"""Fosepel on the CPU: the configuration, the model's structure, the plain functions among themselves, and the engine's
host side (cache slots and state rows of every pass of a repeated span, the kept inputs of the convolutions, batching,
scheduler) over the torch stand-ins of the kernels."""
import copy
import math

import pytest
import torch

import helpers
import fosepel_cases as cases
from plain import fosepel_plain as plain


@pytest.fixture(scope="module")
def fosepel_folders(tmp_path_factory):
    made = {}

    def get(name):
        if name not in made:
            made[name] = cases.make_folder(name, str(tmp_path_factory.mktemp(f"fosepel_{name}")))
        return made[name]
    return get


def test_configuration_reads_every_size_and_round_trips():
    from vt_transformer_b200.config import ConfigError, config_from_dict
    from vt_transformer_b200.config.fosepel import FosepelConfig, FosepelDelta, FosepelMemory
    cfg = config_from_dict(copy.deepcopy(cases.CONFIGS["mix"]))
    assert isinstance(cfg, FosepelConfig) and cfg.vocab == 300 and cfg.width == 64 and len(cfg.layers) == 4
    assert (cfg.norm_eps, cfg.logit_softcap, cfg.loop_start, cfg.loop_stop, cfg.loop_times) == (1e-5, 15.0, 1, 3, 3)
    a = cfg.layers[0].left
    assert (a.flavour, a.heads, a.kv_heads, a.dim, a.vdim, a.scale, a.softcap, a.q_temp_coef, a.q_temp_every) == \
        ("learned_sink", 4, 2, 24, 40, 0.21, 8.0, 0.4, 16)
    m = cfg.layers[0].right
    assert isinstance(m, FosepelMemory) and (m.heads, m.dim, m.vdim, m.gate_cap) == (3, 20, 24, 6.0) and cfg.layers[0].ff == 88
    a = cfg.layers[1].left
    assert (a.flavour, a.heads, a.kv_heads, a.dim, a.vdim, a.rot.dims, a.rot.base) == ("rotary", 4, 1, 32, 16, 16, 3000.0)
    assert (a.rot.scaling.factor, a.rot.scaling.original, a.rot.scaling.fast, a.rot.scaling.slow) == (4.0, 64, 4.0, 1.0)
    d = cfg.layers[2].right
    assert isinstance(d, FosepelDelta) and (d.heads, d.kv_heads, d.dim, d.vdim, d.conv) == (4, 2, 24, 16, 3)
    assert cfg.layers[2].left.flavour == "unit_sink" and cfg.layers[2].ff is None and cfg.layers[3].left.rot.scaling is None
    # the repeated span adds the embedding's output before its first layer in every pass but the first
    assert cfg.run_order() == ((0, False), (1, False), (2, False), (1, True), (2, False), (1, True), (2, False), (3, False))
    assert config_from_dict(cfg.to_dict()) == cfg
    plainer = copy.deepcopy(cases.CONFIGS["wide"])
    assert config_from_dict(plainer).layers[1].left.softcap is None and config_from_dict(plainer).layers[1].left.q_temp_coef is None
    assert config_from_dict(plainer).logit_softcap == 0.0
    for spoil, match in ((lambda c: c["layers"][0].__setitem__("type", "other"), "layers\\[0\\].*'other'"),
                         (lambda c: c["layers"][1]["mixer"].pop("heads"), "layers\\[1\\].mixer.*'heads'"),
                         (lambda c: c["layers"][1]["mixer"]["rot"].__setitem__("dims", 34), "rot.dims"),
                         (lambda c: c["layers"][0]["mixer"]["left"].__setitem__("kv_heads", 3), "kv_heads"),
                         (lambda c: c["layers"][2]["mixer"]["right"].__setitem__("kv_heads", 3), "kv_heads"),
                         (lambda c: c["layers"][2]["mixer"]["right"].__setitem__("conv", 40), "conv"),
                         (lambda c: c["layers"][0]["mixer"]["right"].pop("gate_cap"), "gate_cap"),
                         (lambda c: c["layers"][0]["mlp"].__setitem__("kind", "moe"), "moe"),
                         (lambda c: c["loop"].__setitem__("stop", 9), "loop")):
        bad = copy.deepcopy(cases.CONFIGS["mix"])
        spoil(bad)
        with pytest.raises(ConfigError, match=match):
            config_from_dict(bad)


def test_every_pass_of_a_repeated_span_has_slots_of_its_own():
    from vt_transformer_b200.config import config_from_dict
    from vt_transformer_b200.models.fosepel import fosepel_model_spec
    from vt_transformer_b200.parts.specs import NormedParallelSpec
    spec = fosepel_model_spec(config_from_dict(copy.deepcopy(cases.CONFIGS["mix"])))
    assert [r.block for r in spec.order] == [0, 1, 2, 1, 2, 1, 2, 3]
    assert [r.add_embedding for r in spec.order] == [False, False, False, True, False, True, False, False]
    slots = []
    for r in spec.order:
        slots += list(r.cache) if isinstance(r.cache, tuple) else [r.cache]
    assert slots == list(range(len(slots)))                 # no two runs share a slot
    # the matrix memory beside an attention keeps pages and one state; the delta rule with three taps a state and its last inputs
    assert [len(r.cache) if isinstance(r.cache, tuple) else 1 for r in spec.order] == [2, 1, 3, 1, 3, 1, 3, 1]
    assert isinstance(spec.blocks[0].mixer, NormedParallelSpec) and spec.blocks[0].mixer.scales == (0.5, 0.5)
    assert spec.head.tied_to == "embed" and spec.head.logit_cap == 15.0
    one_tap = fosepel_model_spec(config_from_dict(copy.deepcopy(cases.CONFIGS["wide"])))
    assert len(one_tap.order[-1].cache) == 2                # one tap: nothing of the convolutions is kept


def test_ramped_frequencies_hit_every_branch():
    from vt_transformer_b200.parts.rope import ramped_frequencies
    rot = {"dims": 16, "base": 3000.0, "scaling": {"factor": 4.0, "original": 64, "fast": 4.0, "slow": 1.0}}
    f, m = plain.ramped_frequencies(rot)
    base = [3000.0 ** (-2.0 * i / 16) for i in range(8)]
    assert f[0] == base[0] and f[-1] == pytest.approx(base[-1] / 4.0)      # the fastest pair is kept, the slowest divided
    assert any(base[i] / 4.0 < f[i] < base[i] for i in range(8))            # and some lie between
    assert m == pytest.approx(0.1 * math.log(4.0) + 1.0)
    g, gm = ramped_frequencies(16, 3000.0, (4.0, 64, 4.0, 1.0))
    assert torch.allclose(g.double(), torch.tensor(f, dtype=torch.float64), rtol=1e-6) and gm == pytest.approx(m)
    f0, m0 = plain.ramped_frequencies({"dims": 8, "base": 10.0})
    assert m0 == 1.0 and f0 == [10.0 ** (-2.0 * i / 8) for i in range(4)]


def test_plain_functions_agree_with_their_definitions():
    t = torch.tensor
    # the convolution: zeros before the first token, the last tap is the present token's
    x = t([[1.0], [2.0], [3.0]], dtype=torch.float64)
    w = t([[100.0, 10.0, 1.0]], dtype=torch.float64)
    assert plain.short_convolution(x, w).flatten().tolist() == [1.0, 12.0, 123.0]
    # softmax with a sink of score 0: one key of score 0 gets half of its value
    q = torch.zeros((1, 1, 2), dtype=torch.float64)
    v = t([[[4.0, 8.0]]], dtype=torch.float64)
    assert plain.causal_softmax_attention(q, q, v, 1.0, sink=torch.zeros(1, dtype=torch.float64)).flatten().tolist() == [2.0, 4.0]
    assert plain.causal_softmax_attention(q, q, v, 1.0).flatten().tolist() == [4.0, 8.0]
    # capped scores: a huge score counts as the cap
    q2 = t([[[50.0]], [[50.0]]], dtype=torch.float64)
    k2 = t([[[0.0]], [[1.0]]], dtype=torch.float64)
    v2 = t([[[0.0]], [[1.0]]], dtype=torch.float64)
    got = plain.causal_softmax_attention(q2, k2, v2, 1.0, cap=2.0)[1, 0, 0]
    assert float(got) == pytest.approx(math.exp(2.0 * math.tanh(25.0)) / (1.0 + math.exp(2.0 * math.tanh(25.0))))
    # the delta rule: with beta 1 and no decay a key's value is replaced, not added to
    k = t([[[1.0, 0.0]], [[1.0, 0.0]]], dtype=torch.float64)
    v = t([[[5.0]], [[7.0]]], dtype=torch.float64)
    one = torch.ones((2, 1), dtype=torch.float64)
    assert plain.gated_delta_rule(k, k, v, one, one).flatten().tolist() == [5.0, 7.0]
    assert plain.gated_delta_rule(k, k, v, one * 0.5, one).flatten().tolist() == [2.5, 2.5 + 0.5 * (7.0 - 2.5)]
    # the matrix memory: m starts at 0, so a first token with i = f = -2 is scaled by exp(-2) against a denominator of exp(0)... the max
    q = t([[[1.0]]], dtype=torch.float64)
    o = plain.matrix_memory(q, q, t([[[3.0]]], dtype=torch.float64), t([[-2.0]], dtype=torch.float64), t([[-2.0]], dtype=torch.float64))
    m1 = max(-2.0 + 0.0, -2.0)
    assert float(o) == pytest.approx(3.0 * math.exp(-2.0 - m1) / (max(math.exp(-2.0 - m1), math.exp(-m1)) + 1e-6))


@pytest.mark.parametrize("family", ["whole", "tail", "portions", "mixed"])
def test_cuts_equal_the_plain_implementation(fake_backend, fosepel_folders, family):
    cases.replay(fosepel_folders("mix"), cases.prompts_for("mix"), family, "cpu", "float32")


@pytest.mark.parametrize("name", ["wide", "attention_alone", "parallel_alone", "parallel2_alone", "dense_alone"])
def test_other_sizes_and_each_mechanism_alone(fake_backend, fosepel_folders, name):
    prompts = cases.prompts_for(name, lengths=[1, 12, 45])
    for family in ("whole", "portions", "mixed"):
        cases.replay(fosepel_folders(name), prompts, family, "cpu", "float32", alone=name.endswith("alone"))


def test_portions_shorter_than_the_convolutions_reach(fake_backend, fosepel_folders):
    # five taps keep four inputs: portions of one, two and three tokens shift what is kept instead of replacing it
    cases.replay(fosepel_folders("wide"), cases.prompts_for("wide", lengths=[23, 9]), "portions", "cpu", "float32", sizes=(2, 1, 3, 1, 1, 2))


def test_greedy_generation_through_the_entry_point(fake_backend, fosepel_folders):
    cases.greedy_generation(fosepel_folders("mix"), "mix", "cpu", "float32", n_new=6)


def test_a_tensor_of_the_wrong_shape_is_refused(fake_backend, fosepel_folders, tmp_path):
    from vt_transformer_b200.weights import WeightError

    def spoil(t):
        t["l2.mix.right.q.conv"] = t["l2.mix.right.q.conv"][:, :-1].contiguous()
    with pytest.raises(WeightError):
        cases.runner_for(cases.rewritten(fosepel_folders("mix"), str(tmp_path / "bad"), spoil), "cpu", "float32", num_pages=4)


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
