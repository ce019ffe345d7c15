"""Configurations, weights and scenarios of the Fosepel tests.  Every scenario runs the engine (``ModelRunner.step`` or
``LLM.generate``) and compares with the plain implementation (tests/plain/fosepel_plain.py); each takes the device and
dtype, so the host-side tests run it on the CPU with the stand-in kernels and the GPU tests on cuda:0 with the real ones."""
from __future__ import annotations

import copy
import random
from typing import Dict, List

import numpy as np
import torch

import helpers
from plain import fosepel_plain as plain
from sisetar_cases import rewritten, runner_for, step_all  # noqa: F401  (the same helpers serve every design)


def _rot(dims, base, scaling=None):
    r = {"dims": dims, "base": base}
    if scaling:
        r["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return r


def _dense(ff):
    return None if ff is None else {"kind": "dense", "ff": ff}


def _att(heads, kv_heads, dim, vdim, scale, rot=None, ff=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if rot:
        m["rot"] = rot
    return {"type": "attention", "mixer": m, "mlp": _dense(ff)}


def _par(left, right, ff=None):
    """left: (heads, kv_heads, dim, vdim, scale); right: (heads, kv_heads, dim, vdim, conv)."""
    lt = dict(zip(("heads", "kv_heads", "dim", "vdim", "scale"), left))
    rt = dict(zip(("heads", "kv_heads", "dim", "vdim", "conv"), right))
    return {"type": "parallel", "mixer": {"left": lt, "right": rt}, "mlp": _dense(ff)}


def _par2(left, right, softcap=None, q_temp=None, ff=None):
    """left: (heads, kv_heads, dim, vdim, scale); right: (heads, dim, vdim, gate_cap)."""
    lt = dict(zip(("heads", "kv_heads", "dim", "vdim", "scale"), left))
    if softcap:
        lt["softcap"] = softcap
    if q_temp:
        lt["q_temp"] = {"coef": q_temp[0], "every": q_temp[1]}
    rt = dict(zip(("heads", "dim", "vdim", "gate_cap"), right))
    return {"type": "parallel_2", "mixer": {"left": lt, "right": rt}, "mlp": _dense(ff)}


def _model(vocab, width, layers, loop=None, cap=None, eps=1e-5):
    out = {"architecture": "Fosepel", "vocab": vocab, "width": width, "layers": layers, "norm": {"eps": eps}}
    if loop:
        out["loop"] = dict(zip(("start", "stop", "times"), loop))
    if cap:
        out["logit_softcap"] = cap
    return out


# Configurations that differ from one another in every size and constant: grouped and ungrouped heads and one head, values
# wider and narrower than keys and as wide, a rotation of the whole head, of a part and none, with and without the ramp
# (pairs on all three sides of it), a query temperature whose step lies inside the prompts, with and without capped
# scores, convolutions of 1 to 5 taps, q/k heads of the delta rule shared and not, head sizes of the recurrences that hit
# each shape of the scan (up to 16, up to 32, up to 64, several groups of 64), columns that fill no warp, an inner size of
# the feed-forward that is no multiple of 8, layers without a feed-forward, a repeated span at the start, in the middle,
# over all layers and none, with and without capped logits.
CONFIGS: Dict[str, dict] = {
    "mix": _model(300, 64, [_par2((4, 2, 24, 40, 0.21), (3, 20, 24, 6.0), softcap=8.0, q_temp=(0.4, 16), ff=88),
                            _att(4, 1, 32, 16, 0.19, rot=_rot(16, 3000.0, (4.0, 64, 4.0, 1.0)), ff=100),
                            _par((2, 2, 16, 16, 0.3), (4, 2, 24, 16, 3)),
                            _att(2, 2, 24, 40, 0.25, rot=_rot(24, 100.0), ff=52)],
                  loop=(1, 3, 3), cap=15.0),
    "wide": _model(257, 72, [_par((6, 1, 8, 24, 0.4), (2, 2, 72, 40, 5), ff=52),
                             _par2((1, 1, 40, 8, 0.15), (1, 136, 80, 20.0)),
                             _att(3, 3, 40, 40, 0.16, rot=_rot(8, 1e6, (16.0, 32, 8.0, 2.0))),
                             _par((2, 1, 24, 8, 0.2), (1, 1, 16, 72, 1), ff=40)],
                   loop=(0, 2, 2), eps=1e-6),
    "attention_alone": _model(128, 48, [_att(4, 2, 16, 24, 0.3, rot=_rot(12, 777.0, (6.0, 32, 8.0, 1.0)))], cap=9.0),
    "parallel_alone": _model(128, 48, [_par((3, 1, 16, 8, 0.28), (4, 2, 12, 20, 4))], loop=(0, 1, 2)),
    "parallel2_alone": _model(128, 48, [_par2((2, 1, 24, 16, 0.22), (2, 28, 36, 9.0), softcap=5.0, q_temp=(0.7, 10))]),
    "dense_alone": _model(128, 48, [_att(1, 1, 8, 8, 0.5, ff=60)]),
    # sizes of the kind a served model has: heads of 64 and 128, recurrences with keys of 64 and 128 and values of 128
    "tensor": _model(200, 128, [_par2((4, 2, 64, 64, 0.125), (2, 128, 128, 15.0), softcap=30.0, q_temp=(0.2, 128), ff=256),
                                _att(4, 1, 128, 128, 0.09, rot=_rot(64, 1e4, (4.0, 256, 16.0, 2.0)), ff=96),
                                _par((4, 2, 64, 64, 0.125), (4, 2, 64, 128, 4), ff=96)], loop=(0, 3, 2), cap=30.0),
}
SIGMA = {"mix": 0.15, "wide": 0.12, "attention_alone": 0.25, "parallel_alone": 0.25, "parallel2_alone": 0.25, "dense_alone": 0.2,
         "tensor": 0.1}
SEED = {n: 900 + i for i, n in enumerate(CONFIGS)}
LENGTHS = {"mix": [1, 9, 40, 71, 130], "wide": [3, 33, 90, 152], "attention_alone": [2, 30, 77], "parallel_alone": [1, 25, 66],
           "parallel2_alone": [1, 25, 66], "dense_alone": [4, 19, 50], "tensor": [1, 70, 150, 330, 260]}


def spread_constants(t: Dict[str, torch.Tensor]) -> None:
    """Sinks of the size of a head's largest scores (some above, some below zero), decays between a half and nearly one,
    gates' biases that differ by head: leaving one out, scaling it or giving it to the wrong head then moves the logits far
    beyond rounding."""
    for n in t:
        k = t[n].numel()
        if n.endswith("left.sink"):
            t[n] = torch.linspace(-1.0, 2.5, k).to(t[n].dtype)
        elif n.endswith("right.A_log"):
            t[n] = torch.linspace(-3.5, 0.0, k).to(t[n].dtype)
        elif n.endswith("right.dt_bias"):
            t[n] = torch.linspace(-1.0, 1.0, k).to(t[n].dtype)
        elif n.endswith("right.f.b"):
            t[n] = torch.linspace(1.0, 4.0, k).to(t[n].dtype)
        elif n.endswith("right.i.b"):
            t[n] = torch.linspace(-1.0, 1.5, k).to(t[n].dtype)


def config_of(name: str) -> dict:
    return copy.deepcopy(CONFIGS[name])


def make_folder(name: str, folder: str) -> str:
    from vt_transformer_b200.config import config_from_dict
    from vt_transformer_b200.weights import write_random_model
    made = write_random_model(config_from_dict(config_of(name)), folder + "_raw", seed=SEED[name], sigma=SIGMA[name])
    return rewritten(made, folder, spread_constants)


def prompts_for(name: str, seed: int = 0, lengths=None) -> List[List[int]]:
    rng = random.Random(1700 + seed)
    vocab = CONFIGS[name]["vocab"]
    return [[rng.randrange(vocab) for _ in range(n)] for n in (lengths or LENGTHS[name])]


def tol(dtype: str, ref: torch.Tensor, alone: bool = False) -> float:
    """The bound on |logit - plain logit|, as a part of the spread of the model's plain logits.  32-bit differs by
    rounding and the order of sums only; bfloat16 rounds the activations to 8 bits at every part, less in a model of one
    layer (``alone``) than in a deep one."""
    spread = max(1.0, float(ref.double().std()))
    return (5e-5 if dtype == "float32" else (0.1 if alone else 0.3)) * spread


def outliers_allowed(dtype: str, n: int) -> int:
    """Positions of ``n`` that may lie beyond the bound (and within twice the bound): none in 32-bit; one in fifty (at least
    one) in bfloat16, where now and then a position's logits hang on a sum that rounding moves more than elsewhere (measured:
    the same positions with the plain kernels and with the tensor-core kernels, the others at a seventh of the bound)."""
    return 0 if dtype == "float32" else max(1, n // 50)


def compare(folder, prompts, trace, got, dtype, alone: bool = False) -> float:
    worst, counted, over = 0.0, 0, []
    for n in sorted(trace.expect):
        exp = trace.expect[n]
        assert got[n].shape[0] == len(exp), f"step {n}: {got[n].shape[0]} rows, {len(exp)} wanted"
        for i, (r, pos) in enumerate(exp):
            ref = helpers.plain_logits(folder, prompts[r])
            d = float(np.abs(got[n][i].astype(np.float64) - ref[pos].numpy()).max())
            bound = tol(dtype, ref, alone)
            counted += 1
            assert np.isfinite(d) and d <= 2 * bound, (n, r, pos, d, bound)
            if d > bound:
                over.append(f"step {n}, request {r} (length {len(prompts[r])}), position {pos}: |dlogit| {d:.3e} > {bound:.1e} "
                            f"(entries {[(e['id'], len(e['tokens'])) for e in trace.steps[n]['entries']]})")
            else:
                worst = max(worst, d / bound)
    assert len(over) <= (0 if alone else outliers_allowed(dtype, counted)), over
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
    """Scales the queries of every softmax attention (the norm's weight where q is normed, else the projection and its bias)
    so that a position's weight lies on a few keys: a key that is wrongly seen or hidden, a sink that is left out or a cap
    that is not applied then moves the logits far beyond rounding."""
    for n in list(t):
        if n.endswith("q.norm"):
            t[n] = (t[n].float() * factor).to(t[n].dtype)
        elif n.endswith("left.q") or n.endswith("left.q.b"):
            if n.rsplit(".q", 1)[0] + ".q.norm" not in t:
                t[n] = (t[n].float() * factor).to(t[n].dtype)


def remember_everything(t: Dict[str, torch.Tensor]) -> None:
    """Decays of nearly one, small write strengths and forget gates of nearly one: what the first tokens wrote into a
    recurrent state still decides the output hundreds of tokens later."""
    for n in t:
        if n.endswith("right.A_log"):
            t[n] = torch.full_like(t[n], -7.0)
        elif n.endswith("right.f.b"):
            t[n] = torch.full_like(t[n], 9.0)
        elif n.endswith("right.i.b"):
            t[n] = torch.full_like(t[n], -2.0)


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
        for i, tok in enumerate(o):
            row = ref[len(p) - 1 + i]
            # the token is the plain argmax, or (two logits closer than the rounding) its plain logit is within the bound
            assert float(row.max() - row[tok]) <= 2 * tol(dtype, ref), (len(p), i, tok)
    llm.runner.cache.check()
    assert llm.stats["free_pages"] == [24] * len(llm.runner.cache.groups)
    return outs


def within(got: torch.Tensor, folder, tokens, dtype, alone: bool = False) -> None:
    """``got`` [T, vocab] against the plain logits of ``tokens``, position by position."""
    ref = helpers.plain_logits(folder, tokens)
    assert bool(torch.isfinite(got).all())
    d = (got.double() - ref).abs().max(dim=1).values
    bound = tol(dtype, ref, alone)
    assert float(d.max()) <= 2 * bound and int((d > bound).sum()) <= (0 if alone else outliers_allowed(dtype, len(tokens))), \
        (int(d.argmax()), float(d.max()), bound)
