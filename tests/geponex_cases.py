"""Configurations, weights and scenarios of the Geponex tests.  Every scenario runs the engine (``ModelRunner.step`` or
``LLM.generate``) and compares with the plain implementation (tests/plain/geponex_plain.py); each takes the device and
dtype, so the host-side tests run it on the CPU with the stand-in kernels and the GPU tests on cuda:0 with the real ones."""
from __future__ import annotations

import copy
import random
from typing import Dict, List

import numpy as np
import torch

import helpers
from plain import geponex_plain as plain
from sisetar_cases import rewritten, runner_for, step_all  # noqa: F401  (the same helpers serve every design)


def _rot(dims, base, scaling=None):
    r = {"dims": dims, "base": base}
    if scaling:
        r["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return r


def _lat(heads, dim, rot_dim, vdim, q_rank, kv_rank, scale, base, scaling=None, second=False, mlp=None, weights_of=None):
    out = {"type": "latent_attention_2" if second else "latent_attention",
           "mixer": {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank, "scale": scale,
                     "rot": _rot(rot_dim, base, scaling)}, "mlp": mlp}
    if weights_of is not None:
        out["weights_of"] = weights_of
    return out


def _lig(heads, dim, vdim, decay, mlp=None, weights_of=None):
    out = {"type": "lightning", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "decay": decay}, "mlp": mlp}
    if weights_of is not None:
        out["weights_of"] = weights_of
    return out


def _dense(ff):
    return {"kind": "dense", "ff": ff}


def _moe(experts, top, scale, ff, limit, shared=None):
    return {"kind": "moe", "router": {"experts": experts, "top": top, "scale": scale}, "expert": {"ff": ff, "limit": limit},
            "shared": None if shared is None else {"ff": shared[0], "limit": shared[1]}}


def _model(vocab, width, layers, groups=1, alpha=1.0, eps=1e-5):
    return {"architecture": "Geponex", "vocab": vocab, "width": width, "layers": layers, "norm": {"eps": eps, "groups": groups},
            "postln_alpha": alpha}


# Configurations that differ from one another in every size and constant: values wider and narrower than the plain key
# part and as wide, rotated parts from 4 to 32 dimensions, latents of the queries wider and narrower than the keys' and
# of a size that is no multiple of 8, one head, with and without the ramp over the rotation's frequencies on either
# kind of attention (pairs on both sides of the ramp and inside it), a scale that is not 1 / sqrt(head), norms in 1 to 6
# groups (also groups of 12 values, no multiple of 8), a stream scale of 1 and others, decays of exactly 1 and far below, dense feed-forwards whose inner size
# is no multiple of 8, experts with top of 1 and of all, with and without the shared expert and with a clamp of its own,
# layers without a feed-forward, layers that use an earlier layer's weights (of each kind of mixer, more than once).
_M1 = _moe(5, 2, 2.0, 20, 1.5, shared=(36, 3.0))
_D1 = _dense(100)
CONFIGS: Dict[str, dict] = {
    "mix": _model(300, 64, [_lig(3, 24, 40, [0.7, 0.95, 1.0], mlp=_M1),
                            _lat(3, 24, 16, 40, 40, 48, 0.2, 3000.0, scaling=(8.0, 64, 4.0, 1.0), mlp=_D1),
                            _lat(2, 16, 8, 16, 24, 32, 0.3, 100.0, second=True),
                            _lat(3, 24, 16, 40, 40, 48, 0.2, 3000.0, scaling=(8.0, 64, 4.0, 1.0), mlp=_D1, weights_of=1),
                            _lig(3, 24, 40, [0.7, 0.95, 1.0], mlp=_M1, weights_of=0),
                            _lat(4, 8, 32, 8, 16, 24, 0.17, 5e4, scaling=(3.0, 40, 2.0, 0.5), second=True, mlp=_moe(6, 1, 0.8, 24, 0.9))],
                  groups=4, alpha=2.5),
    "wide": _model(257, 72, [_lat(1, 40, 4, 24, 12, 20, 0.11, 7.0, second=True, mlp=_moe(4, 4, 1.0, 40, 2.5, shared=(24, 1.0))),
                             _lig(2, 72, 16, [0.99, 0.5], mlp=_dense(52)),
                             _lat(6, 16, 24, 72, 64, 40, 0.25, 1e6, mlp=_moe(3, 2, 1.7, 12, 4.0)),
                             _lig(2, 72, 16, [0.99, 0.5], mlp=_dense(52), weights_of=1),
                             _lig(2, 72, 16, [0.99, 0.5], mlp=_dense(52), weights_of=3)],
                   groups=6, alpha=1.0, eps=1e-6),
    "latent_alone": _model(128, 48, [_lat(4, 16, 8, 24, 24, 32, 0.22, 777.0, scaling=(6.0, 32, 8.0, 1.0))], groups=2, alpha=1.6),
    "latent2_alone": _model(128, 48, [_lat(3, 8, 16, 16, 40, 24, 0.27, 300.0, second=True)], groups=3, alpha=0.7),
    "lightning_alone": _model(128, 48, [_lig(3, 20, 28, [0.8, 0.95, 0.99])], groups=1, alpha=1.3),
    "dense_alone": _model(128, 48, [_lig(1, 8, 8, [0.5], mlp=_dense(60))], groups=6, alpha=2.0),
    "experts_alone": _model(128, 48, [_lig(1, 8, 8, [0.5], mlp=_moe(7, 3, 1.4, 28, 1.2, shared=(12, 0.6)))], groups=2, alpha=0.9),
    # sizes of the kind a served model has: a latent of 128 with a rotated part of 32 beside it, heads of 64 and 32
    "tensor": _model(200, 128, [_lat(8, 32, 32, 64, 48, 128, 0.12, 1e4, scaling=(4.0, 256, 16.0, 2.0), mlp=_moe(3, 3, 1.2, 24, 2.0, shared=(16, 2.0))),
                                _lat(4, 64, 32, 32, 64, 128, 0.1, 5e5, second=True, mlp=_dense(96)),
                                _lig(4, 32, 64, [0.9, 0.97, 0.995, 1.0]),
                                _lat(4, 64, 32, 32, 64, 128, 0.1, 5e5, second=True, mlp=_dense(96), weights_of=1)], groups=2, alpha=1.8),
}
SIGMA = {"mix": 0.15, "wide": 0.12, "latent_alone": 0.25, "latent2_alone": 0.25, "lightning_alone": 0.2, "dense_alone": 0.2, "experts_alone": 0.2,
         "tensor": 0.1}
SEED = {n: 700 + i for i, n in enumerate(CONFIGS)}
LENGTHS = {"mix": [1, 9, 40, 71, 130], "wide": [3, 33, 90, 152], "latent_alone": [2, 30, 77], "latent2_alone": [1, 25, 66],
           "lightning_alone": [1, 25, 66], "dense_alone": [4, 19, 50], "experts_alone": [4, 19, 50], "tensor": [1, 70, 150, 330, 260]}


def every_expert(name: str) -> str:
    """The name of the configuration ``name`` with every router's ``top`` set to its number of experts."""
    return name + "+all"


def for_dtype(name: str, dtype: str) -> str:
    """The configuration that a test of the whole model runs in ``dtype``.  In bfloat16 the rounding of the activations
    decides a router's close call the other way now and then; the token then runs other experts, and through latents and
    states every later position of a deep model moves by more than rounding explains.  So the deep models run in bfloat16
    with every expert chosen (the weights still come from the scores), and the choice among experts is tested in 32-bit
    on the same kernels and in bfloat16 on the model of one layer, where a close call touches its own position only and
    is left out."""
    return name if dtype == "float32" else every_expert(name)


def _base(name: str) -> str:
    return name[:-len("+all")] if name.endswith("+all") else name


def config_of(name: str) -> dict:
    cfg = copy.deepcopy(CONFIGS[_base(name)])
    if name.endswith("+all"):
        for layer in cfg["layers"]:
            if layer["mlp"] is not None and layer["mlp"]["kind"] == "moe":
                layer["mlp"]["router"]["top"] = layer["mlp"]["router"]["experts"]
    return cfg


def spread_sinks(t: Dict[str, torch.Tensor]) -> None:
    """Sinks of the size of a head's largest scores (some above, some below zero), so that leaving one out, scaling it or
    counting it for every key would move the logits far beyond rounding."""
    for n in t:
        if n.endswith("mix.sink"):
            t[n] = torch.linspace(-1.0, 2.5, t[n].numel()).to(t[n].dtype)


def make_folder(name: str, folder: str) -> str:
    from vt_transformer_b200.config import config_from_dict
    from vt_transformer_b200.weights import write_random_model
    made = write_random_model(config_from_dict(config_of(name)), folder + "_raw", seed=SEED[_base(name)], sigma=SIGMA[_base(name)])
    return rewritten(made, folder, spread_sinks)


def prompts_for(name: str, seed: int = 0, lengths=None) -> List[List[int]]:
    name = _base(name)
    rng = random.Random(1300 + seed)
    vocab = CONFIGS[name]["vocab"]
    return [[rng.randrange(vocab) for _ in range(n)] for n in (lengths or LENGTHS[name])]


def tol(dtype: str, ref: torch.Tensor, alone: bool = False) -> float:
    """The bound on |logit - plain logit|, as a part of the spread of the model's plain logits.  32-bit differs by
    rounding and the order of sums only; bfloat16 rounds the activations to 8 bits at every part, less in a model of one
    layer (``alone``) than in a deep one."""
    spread = max(1.0, float(ref.double().std()))
    return (5e-5 if dtype == "float32" else (0.1 if alone else 0.35)) * spread


def outliers_allowed(dtype: str, n: int) -> int:
    """Positions of ``n`` that may lie beyond the bound: none in 32-bit, one in fifty (at least one) in bfloat16."""
    return 0 if dtype == "float32" else max(1, n // 50)


_close = {}
CLOSE_CALL = 0.03       # a router's margin, as a part of its largest logit, below which bfloat16 rounding may choose otherwise


def close_calls(folder, tokens, dtype) -> set:
    """The positions at which a router of the plain model makes a close call.  Comparisons in bfloat16 leave these
    positions out; in 32-bit every position counts."""
    if dtype == "float32":
        return set()
    key = (folder, tuple(tokens))
    if key not in _close:
        margins = []
        plain.forward(plain.read_config(folder), helpers._plain_weights(folder), list(tokens), margins=margins)
        found = set()
        for m in margins:
            found |= set(int(i) for i in torch.nonzero(m < CLOSE_CALL).flatten())
        _close[key] = found
    return _close[key]


def within(got: torch.Tensor, folder, tokens, dtype, alone: bool = False) -> None:
    """``got`` [T, vocab] against the plain logits of ``tokens``, position by position except at close calls."""
    ref = helpers.plain_logits(folder, tokens)
    keep = [i for i in range(len(tokens)) if i not in close_calls(folder, tokens, dtype)]
    assert bool(torch.isfinite(got).all()) and 3 * len(keep) >= len(tokens)
    d = (got[keep].double() - ref[keep]).abs().max(dim=1).values
    over = int((d > tol(dtype, ref, alone)).sum())
    assert over <= (0 if alone else outliers_allowed(dtype, len(keep))), (over, float(d.max()), tol(dtype, ref, alone))


def compare(folder, prompts, trace, got, dtype, alone: bool = False) -> float:
    worst, counted, total, over = 0.0, 0, 0, []
    for n in sorted(trace.expect):
        exp = trace.expect[n]
        assert got[n].shape[0] == len(exp), f"step {n}: {got[n].shape[0]} rows, {len(exp)} wanted"
        for i, (r, pos) in enumerate(exp):
            ref = helpers.plain_logits(folder, prompts[r])
            total += 1
            if pos in close_calls(folder, prompts[r], dtype):
                assert np.isfinite(got[n][i]).all()
                continue
            counted += 1
            d = float(np.abs(got[n][i].astype(np.float64) - ref[pos].numpy()).max())
            bound = tol(dtype, ref, alone)
            assert np.isfinite(d)
            if d > bound:
                over.append(f"step {n}, request {r} (length {len(prompts[r])}), position {pos}: |dlogit| {d:.3e} > {bound:.1e} "
                            f"(entries {[(e['id'], len(e['tokens'])) for e in trace.steps[n]['entries']]})")
            else:
                worst = max(worst, d / bound)
    assert len(over) <= (0 if alone else outliers_allowed(dtype, counted)), over
    assert 3 * counted >= total, f"only {counted} of {total} positions are free of a router's close call: the test compares too little"
    return worst


def replay(folder, prompts, family, device, dtype, page_size=16, sizes=None, tail=20, alone: bool = False) -> float:
    """One way of cutting the requests into steps, with no more pages than the live requests need (so that pages and
    state rows are used again), against the plain implementation.  Returns the worst error as a part of its bound."""
    make = {"whole": helpers.trace_whole, "tail": lambda p: helpers.trace_tail(p, tail=tail),
            "portions": (lambda p: helpers.trace_portions(p, sizes=sizes)) if sizes else helpers.trace_portions,
            "mixed": lambda p: helpers.trace_mixed(p, max_live=3, seed=5)}[family]
    trace = make(prompts)
    pages = max(1, helpers.tokens_needed(trace, round_to=page_size) // page_size)
    runner = runner_for(folder, device, dtype, num_pages=pages, max_requests=3 if family == "mixed" else 1, page_size=page_size)
    got = helpers.run_trace_inproc(runner, trace)
    worst = compare(folder, prompts, trace, got, dtype, alone)
    assert runner.cache.free_pages() == [g.pool.num_pages for g in runner.cache.groups]
    assert runner.cache.free_rows == runner.cache.max_requests
    runner.cache.check()
    return worst


def sharpen_attention(t: Dict[str, torch.Tensor], factor: float = 4.0) -> None:
    """Scales the weights of the norms of the queries' latents so that a position's attention lies on a few keys: a key
    that is wrongly seen or wrongly hidden then moves the logits far beyond rounding."""
    for n in t:
        if n.endswith("mix.dq.norm"):
            t[n] = (t[n].float() * factor).to(t[n].dtype)


def greedy_generation(folder, name, device, dtype, n_new=12):
    """Greedy generation through the entry point and its scheduler (portions of prompts beside decoding requests)."""
    from vt_transformer_b200 import LLM, SamplingParams
    prompts = prompts_for(name)[1:4]
    llm = LLM(folder, dtype=dtype, device=device, max_running_reqs=3, num_pages=24, max_seq_len=192, page_size=16,
              max_extend_tokens=40, chunk_size=24)
    outs = llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=n_new, ignore_eos=True))
    cfg, w = plain.read_config(folder), helpers._plain_weights(folder)
    for p, o in zip(prompts, outs):
        assert len(o) == n_new
        ref = plain.forward(cfg, w, list(p) + o)
        close = close_calls(folder, list(p) + o, dtype)
        for i, tok in enumerate(o):
            if len(p) - 1 + i in close:
                continue
            row = ref[len(p) - 1 + i]
            # the token is the plain argmax, or (two logits closer than the rounding) its plain logit is within the bound
            assert float(row.max() - row[tok]) <= 2 * tol(dtype, ref), (len(p), i, tok)
    llm.runner.cache.check()
    assert llm.stats["free_pages"] == [24] * len(llm.runner.cache.groups)
    return outs
