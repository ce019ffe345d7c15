"""Geponex on the GPU: the kernels against the plain functions, every mechanism alone and the whole model, through the
engine's step and entry point, against the plain implementation (tests/plain/geponex_plain.py)."""
import math

import pytest
import torch

import helpers
import geponex_cases as cases
from plain import geponex_plain as plain

pytestmark = pytest.mark.gpu
DTYPES = ["bfloat16", "float32"]
DEV = "cuda:0"
F = torch.float64


@pytest.fixture(scope="module")
def geponex_folders(tmp_path_factory):
    made = {}

    def get(name):
        if name not in made:
            made[name] = cases.make_folder(name, str(tmp_path_factory.mktemp(f"geponex_{name}")))
        return made[name]
    return get


def _logits(folder, tokens):
    return helpers.plain_logits(folder, tokens)


# ----------------------------------------------------------------------------- kernels against the plain functions


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("width", [48, 200, 4104])
def test_token_shift_kernel_carries_the_row_before(dtype, width):
    """Two sequences in a step (one continues from its row of state, one starts), then a second step of single tokens."""
    from vt_transformer_b200 import ops
    g = torch.Generator().manual_seed(width)
    mu = torch.rand(width, generator=g)
    state = torch.zeros((3, width))
    state[2] = torch.randn(width, generator=g)
    before = {0: state[2].double().clone(), 1: torch.zeros(width, dtype=F)}
    rows = [2, 0]
    sd = state.to(DEV)
    for lens in ([5, 3], [1, 1], [2, 1]):
        x = torch.randn((sum(lens), width), generator=g)
        ctx = helpers.step_context(lens, [0] * len(lens), DEV)
        ctx.rows = torch.tensor(rows, dtype=torch.int32, device=DEV)
        out = torch.empty((sum(lens), width), dtype=dtype, device=DEV)
        ops.token_shift(x.to(DEV), mu.to(DEV), sd, ctx, out)
        at = 0
        for s, n in enumerate(lens):
            ref, before[s] = plain.token_shift(x[at:at + n].double(), before[s], mu.double())
            assert float((out[at:at + n].double().cpu() - ref).abs().max()) <= (1e-6 if dtype == torch.float32 else 4e-2)
            assert torch.equal(sd[rows[s]].cpu(), x[at + n - 1])
            at += n
    assert torch.equal(sd[1].cpu(), torch.zeros(width))


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("width,groups", [(48, 1), (48, 3), (200, 5), (4096, 2), (4104, 1), (72, 6), (200, 50)])
def test_norm_kernel_in_groups_after_the_scaled_sum(dtype, width, groups):
    """x <- norm(a x + delta) in groups, the unrounded result back into the stream and a rounded copy for the next part."""
    from vt_transformer_b200 import ops
    g = torch.Generator().manual_seed(width + groups)
    x = torch.randn((7, width), generator=g) * 3
    w = 1 + 0.2 * torch.randn(width, generator=g)
    delta = (torch.randn((7, width), generator=g) * 2).to(dtype)
    xd, out = x.to(DEV), torch.empty((7, width), dtype=dtype, device=DEV)
    ops.rmsnorm(xd, w.to(DEV), 1e-5, out, delta=delta.to(DEV), groups=groups, x_scale=1.7, to_stream=True)
    ref = plain.grouped_rms_norm(1.7 * x.double() + delta.double(), w.double(), 1e-5, groups)
    assert float((xd.double().cpu() - ref).abs().max()) <= 2e-5
    assert float((out.double().cpu() - ref).abs().max()) <= (2e-5 if dtype == torch.float32 else 4e-2)
    if dtype == torch.bfloat16:
        assert torch.equal(out.cpu(), xd.cpu().to(torch.bfloat16))


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_activation_kernels(dtype):
    from vt_transformer_b200 import ops
    g = torch.Generator().manual_seed(11)
    p, q = torch.tensor(0.3, dtype=F), torch.tensor(-0.4, dtype=F)
    sp = torch.nn.functional.softplus
    for shape in ((9, 40), (9, 41), (300, 1024)):            # eight values a thread, and one where the count is no multiple of 8
        z = (torch.randn(shape, generator=g) * 3).to(dtype)
        out = torch.empty_like(z, device=DEV)
        ops.xielu(z.to(DEV), out, float(sp(p)), float(0.5 + sp(q)))
        ref = plain.xielu(z.double(), p, q)
        assert float(((out.double().cpu() - ref).abs() / (1 + ref.abs())).max()) <= (1e-6 if dtype == torch.float32 else 8e-3)
    # gate and up side by side and in alternating runs of 8, with a second clamp from a column on
    n, split = 48, 32
    gate, up = (torch.randn((9, n), generator=g) * 2).to(dtype), (torch.randn((9, n), generator=g) * 2).to(dtype)
    one = torch.eye(n, dtype=F)
    ref = torch.cat([plain.expert(torch.eye(1, dtype=F), gate[t:t + 1, :split].double().T, up[t:t + 1, :split].double().T, one[:split, :split], 1.5)
                     for t in range(9)])
    ref2 = torch.cat([plain.expert(torch.eye(1, dtype=F), gate[t:t + 1, split:].double().T, up[t:t + 1, split:].double().T, one[split:, split:], 0.6)
                      for t in range(9)])
    ref = torch.cat([ref, ref2], dim=1)
    for interleave in (0, 8):
        gu = torch.cat([gate, up], dim=1) if not interleave else torch.stack([gate.view(9, -1, 8), up.view(9, -1, 8)], dim=2).reshape(9, -1)
        out = torch.empty((9, n), dtype=dtype, device=DEV)
        ops.gate_clamp(gu.to(DEV), out, interleave, 1.702, 1.5, split=split, limit2=0.6)
        assert float((out.double().cpu() - ref).abs().max()) <= (2e-6 if dtype == torch.float32 else 3e-2)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("heads,v_dim", [(1, 84), (1, 1100), (2, 2048), (3, 40)])
def test_heads_normed_together_and_gated(dtype, heads, v_dim):
    """The heads' results normed as one vector with a weight a channel, times sigmoid(gate): narrow heads (a warp each) and
    wide ones (a CTA each); the row of a padding token becomes zero."""
    from vt_transformer_b200 import ops
    g = torch.Generator().manual_seed(v_dim)
    T = 6
    o = torch.randn((T, heads * v_dim), generator=g) * 3
    y = torch.randn((T, 16 + heads * v_dim), generator=g).to(dtype)
    w = 1 + 0.2 * torch.randn(heads * v_dim, generator=g)
    seq = torch.tensor([0, 0, 1, -1, 2, 2], dtype=torch.int32)
    out = torch.full((T, 8 + heads * v_dim), 5.0, dtype=dtype, device=DEV)
    ops.head_norm_gate(o.to(DEV), y.to(DEV), 16, w.to(DEV), True, 1e-5, "sigmoid", out, 8, 1.0, heads, v_dim, token_seq=seq.to(DEV))
    ref = torch.cat([plain.rms_norm(o[:, h * v_dim:(h + 1) * v_dim].double(), w[h * v_dim:(h + 1) * v_dim].double(), 1e-5) for h in range(heads)], dim=1)
    ref = ref * torch.sigmoid(y[:, 16:].double())
    ref[3] = 0
    assert float((out[:, 8:].double().cpu() - ref).abs().max()) <= (2e-5 if dtype == torch.float32 else 4e-2)
    assert float((out[:, :8].float().cpu() - 5.0).abs().max()) == 0


@pytest.mark.parametrize("experts,top", [(5, 2), (1, 1), (40, 40), (130, 7), (3, 1)])
def test_routing_kernel_with_sigmoid_scores(experts, top):
    """Rows that point along router rows, so that no choice is a close call: the picks are those of the plain routing and
    the weights their sigmoid scores over the picks' sum, scaled."""
    from vt_transformer_b200 import ops
    g = torch.Generator().manual_seed(experts)
    T, width = 9, 64
    router = torch.randn((experts, width), generator=g)
    order = [[(3 * t + 5 * k) % experts for k in range(experts)] for t in range(T)]
    x = torch.stack([sum((top + 2.0 - min(k, top + 1)) * router[order[t][k]] / router[order[t][k]].norm() ** 2 for k in range(min(top + 1, experts)))
                     for t in range(T)])
    ids, wts = torch.empty((T, top), dtype=torch.int32, device=DEV), torch.empty((T, top), device=DEV)
    ops.route_topk(None, top, ids, wts, x=x.to(DEV), router=router.to(DEV), weights_by="sigmoid_share", scale=1.3)
    want_ids, want_w = plain.route(x.double(), router.double(), top, 1.3)
    if experts > top + 1:
        assert torch.equal(ids.cpu().long(), want_ids)
        assert float((wts.double().cpu() - want_w).abs().max()) <= 1e-5
    else:
        assert torch.equal(ids.cpu().long().sort(dim=1).values, want_ids.sort(dim=1).values)
        assert float((wts.double().cpu().sum(1) - 1.3).abs().max()) <= 1e-5


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("tokens", [5, 150])
@pytest.mark.parametrize("heads,inner,outer,tail", [(3, 24, 48, 16), (2, 128, 136, 32), (5, 40, 8, 8), (1, 200, 264, 0)])
def test_products_of_the_heads(dtype, tokens, heads, inner, outer, tail):
    """out[t, h] = x[t, h] M_h, with the rotated tail copied behind a head's outputs, and with the sigmoid gate: a few tokens
    (the plain kernel) and many (bfloat16: the tensor cores)."""
    from vt_transformer_b200 import ops
    g = torch.Generator().manual_seed(inner + outer)
    x = torch.randn((tokens, heads, inner + tail), generator=g).to(dtype)
    m = (torch.randn((heads, inner, outer), generator=g) / math.sqrt(inner)).to(dtype)
    gate = torch.randn((tokens, 8 + heads * outer), generator=g).to(dtype)
    freq, mult = plain.rotary_frequencies(max(tail, 2), 300.0, {"factor": 4.0, "original": 16, "fast": 4.0, "slow": 1.0})
    ctx = helpers.step_context([tokens - 2, 2], [7, 0], DEV)
    positions = torch.cat([torch.arange(7, 7 + tokens - 2), torch.arange(2)])
    ref = torch.einsum("thi,hio->tho", x[..., :inner].double(), m.double())
    tol = 2e-5 if dtype == torch.float32 else 3e-2
    xd, md = x.view(tokens, -1).to(DEV), m.to(DEV)
    out = torch.zeros((tokens, 8 + heads * (outer + tail)), dtype=dtype, device=DEV)
    if tail:
        ops.head_matmul(xd, 0, inner + tail, md, out, 8, outer + tail, mode="rotated_tail", tail=tail, frequencies=freq.float().to(DEV),
                        mult=mult, ctx=ctx)
        turned = plain.rotate_interleaved(x[..., inner:].double(), positions, freq, mult)
        got = out[:, 8:].double().cpu().view(tokens, heads, outer + tail)
        assert float((got[..., :outer] - ref).abs().max()) <= tol and float((got[..., outer:] - turned).abs().max()) <= tol
    else:
        ops.head_matmul(xd, 0, inner, md, out, 8, outer)
        assert float((out[:, 8:].double().cpu().view(tokens, heads, outer) - ref).abs().max()) <= tol
    assert float(out[:, :8].abs().max()) == 0
    out2 = torch.empty((tokens, heads * outer), dtype=dtype, device=DEV)
    ops.head_matmul(xd, 0, inner + tail, md, out2, 0, outer, mode="gate", gate=gate.to(DEV), gate_col=8)
    want = ref * torch.sigmoid(gate[:, 8:].double()).view(tokens, heads, outer)
    assert float((out2.double().cpu().view(tokens, heads, outer) - want).abs().max()) <= tol


@pytest.mark.parametrize("sink", [False, True])
@pytest.mark.parametrize("heads,key,v_dim,page", [(5, 80, 64, 16), (6, 176, 128, 64), (3, 48, 16, 16), (16, 320, 256, 64), (6, 576, 512, 32),
                                                  (70, 64, 32, 16), (5, 112, 80, 16)])
def test_latent_attention_kernel_on_the_tensor_cores(heads, key, v_dim, page, sink):
    """Rows that all heads share, their first numbers the values: a sequence that goes on from 37 cached tokens beside one
    that starts, over shuffled pages; then a step of single tokens.  Against the plain softmax attention."""
    from vt_transformer_b200 import ops
    assert ops.backend().attention_latent_supports(key, v_dim)
    g = torch.Generator().manual_seed(heads + key)
    scale = 1.7 / math.sqrt(key)
    sinks = torch.linspace(-1.0, 2.0, heads) if sink else None
    lengths = [37 + 70 + 1, 5 + 1]
    rows = [torch.randn((n, key), generator=g).to(torch.bfloat16) for n in lengths]
    n_pages = sum(-(-n // page) for n in lengths) + 3
    order = torch.randperm(n_pages, generator=g).tolist()
    pages = torch.zeros((n_pages, 1, page, key), dtype=torch.bfloat16)
    table = torch.full((2, max(-(-n // page) for n in lengths)), -1, dtype=torch.int32)
    for s, r in enumerate(rows):
        for j in range(-(-len(r) // page)):
            table[s, j] = order.pop()
            part = r[j * page:(j + 1) * page]
            pages[table[s, j], 0, :len(part)] = part
    pd, td = pages.to(DEV), table.to(DEV)
    for q_lens, starts in (([70, 5], [37, 0]), ([1, 1], [107, 5])):
        T = sum(q_lens)
        q = torch.randn((T, heads, key), generator=g).to(torch.bfloat16)
        ctx = helpers.step_context(q_lens, starts, DEV)
        out = torch.full((T, heads * v_dim), 7.0, dtype=torch.bfloat16, device=DEV)
        before = ops.launches
        ops.attention_latent(q.view(T, -1).to(DEV), 0, out, 0, pd, ctx, td, heads, key, v_dim, scale, sinks=None if sinks is None else sinks.to(DEV))
        assert ops.launches == before + 1
        at = 0
        for s, (n, start) in enumerate(zip(q_lens, starts)):
            k = rows[s][:start + n].double()
            ref = plain.softmax_attention(q[at:at + n].double(), k[:, None, :].expand(-1, heads, -1), k[:, None, :v_dim].expand(-1, heads, -1),
                                          torch.arange(start, start + n), scale, None if sinks is None else sinks.double())
            got = out[at:at + n].double().cpu().view(n, heads, v_dim)
            assert float((got - ref).abs().max()) <= 2.5e-2, (q_lens, s)
            at += n


# ----------------------------------------------------------------------------- each mechanism alone, in a model of one layer


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["latent_alone", "latent2_alone", "lightning_alone", "dense_alone", "experts_alone"])
def test_each_mechanism_alone(geponex_folders, name, dtype):
    folder = geponex_folders(name)
    prompts = cases.prompts_for(name, lengths=[1, 12, 45])
    for family in ("whole", "tail", "portions"):
        cases.replay(folder, prompts, family, DEV, dtype, alone=name != "experts_alone")


def test_the_sink_counts_once_and_unscaled(geponex_folders, tmp_path):
    """The plain logits without the sinks, and with sinks multiplied by the attention's scale, differ from the model's far
    beyond the bound (so a kernel that drops or scales the sink would show), and the engine gives the model's."""
    folder = geponex_folders("latent2_alone")
    ids = cases.prompts_for("latent2_alone", lengths=[40])[0]
    ref = _logits(folder, ids)

    def no_sink(t):
        t["l0.mix.sink"] = torch.full_like(t["l0.mix.sink"], -30.0)

    def scaled_sink(t):
        t["l0.mix.sink"] = (t["l0.mix.sink"].float() * cases.CONFIGS["latent2_alone"]["layers"][0]["mixer"]["scale"]).to(t["l0.mix.sink"].dtype)
    for n, change in (("none", no_sink), ("scaled", scaled_sink)):
        other = _logits(cases.rewritten(folder, str(tmp_path / n), change), ids)
        assert float((other - ref).abs().max()) > 3 * cases.tol("bfloat16", ref, alone=True)
    for dtype in DTYPES:
        runner = cases.runner_for(folder, DEV, dtype, num_pages=4, max_requests=1)
        for cuts in ([40], [30, 1], [2]):
            row = runner.admit()
            got = cases.step_all(runner, row, ids, cuts)
            runner.release(row)
            assert float((got - ref).abs().max()) <= cases.tol(dtype, ref, alone=True)


# ----------------------------------------------------------------------------- the whole model, cut in every way


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["mix", "wide", "tensor"])
@pytest.mark.parametrize("family", ["whole", "tail", "portions", "mixed"])
def test_cuts_equal_the_plain_implementation(geponex_folders, name, family, dtype):
    page = 64 if name == "tensor" else 16
    cases.replay(geponex_folders(cases.for_dtype(name, dtype)), cases.prompts_for(name), family, DEV, dtype, page_size=page,
                 tail=70 if name == "tensor" else 20, sizes=(40, 3, 64, 2, 150) if name == "tensor" else None)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["mix", "experts_alone"])
def test_tokens_grouped_by_expert(geponex_folders, monkeypatch, name, dtype):
    """Portions with many picks group their tokens by expert instead of running every expert on every token: forced here
    for every portion, also those in which an expert gets no token."""
    from vt_transformer_b200 import ops
    monkeypatch.setattr(ops, "EXPERTS_GROUPED_MIN_PICKS", 1)
    folder = geponex_folders(cases.for_dtype(name, dtype) if name != "experts_alone" else name)
    for family in ("whole", "portions", "mixed"):
        cases.replay(folder, cases.prompts_for(name), family, DEV, dtype)


@pytest.mark.parametrize("dtype", DTYPES)
def test_portions_of_two_tokens_and_pages_of_64(geponex_folders, dtype):
    folder = geponex_folders(cases.for_dtype("mix", dtype))
    cases.replay(folder, cases.prompts_for("mix")[1:4], "portions", DEV, dtype, sizes=(2,))
    cases.replay(folder, cases.prompts_for("mix"), "mixed", DEV, dtype, page_size=64)
    cases.replay(folder, cases.prompts_for("mix"), "tail", DEV, dtype, page_size=64, tail=40)


@pytest.mark.parametrize("dtype", DTYPES)
def test_batches_of_unequal_requests_equal_each_alone_and_rows_are_used_again(geponex_folders, dtype):
    """Three requests of different lengths stepped together, one of them sitting a step out; then the same rows and
    pages serve other requests.  In 32-bit the logits are those of each request alone, bit for bit."""
    from vt_transformer_b200.engine.batch import StepEntry
    folder = geponex_folders(cases.for_dtype("mix", dtype))
    runner = cases.runner_for(folder, DEV, dtype, num_pages=16, max_requests=3)
    for turn in range(2):
        prompts = cases.prompts_for("mix", seed=turn, lengths=[50, 7, 23])
        alone = []
        for p in prompts:
            row = runner.admit()
            alone.append(cases.step_all(runner, row, p, [len(p)]))
            runner.release(row)
        rows = [runner.admit() for _ in prompts]
        done, got = [0, 0, 0], [[], [], []]
        step = 0
        while any(d < len(p) for d, p in zip(done, prompts)):
            entries, who = [], []
            for i, p in enumerate(prompts):
                if done[i] < len(p) and not (i == 1 and step == 1):
                    k = min([9, 1, 4][(i + step) % 3], len(p) - done[i])
                    entries.append(StepEntry(rows[i], p[done[i]:done[i] + k], list(range(k))))
                    who.append((i, k))
                    done[i] += k
            logits, at = runner.step(entries).double().cpu(), 0
            for i, k in who:
                got[i].append(logits[at:at + k])
                at += k
            step += 1
        runner.check_status()
        for i, p in enumerate(prompts):
            cases.within(torch.cat(got[i]), folder, p, dtype)
            if dtype == "float32":
                assert torch.equal(torch.cat(got[i]), alone[i]), "logits depend on what else is in the batch"
        for r in rows:
            runner.release(r)
        runner.cache.check()


# ----------------------------------------------------------------------------- far keys, page borders, the first tokens


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["latent_alone", "latent2_alone"])
def test_a_key_hundreds_of_tokens_back_and_at_page_borders(geponex_folders, tmp_path, name, dtype):
    """Latent attention alone, sharpened so that one key can carry a position's weight: a marked token at position 3, at a
    page's last place and at the next page's first decides the logits at position 389, across 24 pages; whole, in portions,
    and with the asking tokens decoded one by one."""
    folder = cases.rewritten(geponex_folders(name), str(tmp_path / "far"), lambda t: cases.sharpen_attention(t, 4.0))
    base = cases.prompts_for(name, lengths=[392])[0]
    plain_base = _logits(folder, base)
    # queries four times as long make the scores' rounding in bfloat16 four times as large: twice the bound of a model of
    # one layer there (the marked key still moves the logits by more than three times as much)
    bound = cases.tol(dtype, plain_base, alone=True) * (2.0 if dtype == "bfloat16" else 1.0)
    runner = cases.runner_for(folder, DEV, dtype, num_pages=26, max_requests=1)
    for where in (3, 15, 16, 383):
        best = (0.0, 0, 0)
        for tok in range(0, 128, 2):                    # the token and the asking position (decoded alone below) that show it best
            ids = list(base)
            ids[where] = tok
            d = (_logits(folder, ids)[384:] - plain_base[384:]).abs().max(dim=1).values
            best = max(best, (float(d.max()), tok, 384 + int(d.argmax())))
        assert best[0] > 3 * bound, (where, best)
        ids = list(base)
        ids[where] = best[1]
        ref = _logits(folder, ids)
        for cuts in ([len(ids)], [150, 37, 190] + [1] * 15, [380] + [1] * 12):
            row = runner.admit()
            got = cases.step_all(runner, row, ids, cuts)
            runner.release(row)
            assert float((got - ref).abs().max()) <= bound, (where, cuts)


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_token_far_back_still_decides_a_lightning_state(geponex_folders, tmp_path, dtype):
    """Decays of nearly one and of one: what token 2 wrote into the state decides the logits 400 tokens later.  The
    prompt runs in portions, its end token by token; the plain logits with another token 2 differ far beyond the bound."""
    def slow(c):
        c["layers"][0]["mixer"]["decay"] = [0.999, 1.0, 0.9995]
    folder = cases.rewritten(geponex_folders("lightning_alone"), str(tmp_path / "long"), lambda t: None, config=slow)
    ids = cases.prompts_for("lightning_alone", lengths=[420])[0]
    other = list(ids)
    other[2] = (ids[2] + 17) % 128
    ref, ref_other = _logits(folder, ids), _logits(folder, other)
    assert float((ref[-1] - ref_other[-1]).abs().max()) > 100 * cases.tol("float32", ref)
    runner = cases.runner_for(folder, DEV, dtype, num_pages=1, max_requests=2)
    for tokens, want in ((ids, ref), (other, ref_other)):
        row = runner.admit()
        got = cases.step_all(runner, row, tokens, [150, 37, 200] + [1] * 40)
        runner.release(row)
        assert float((got - want).abs().max()) <= cases.tol(dtype, want, alone=True)


@pytest.mark.parametrize("dtype", DTYPES)
def test_the_shifted_row_of_a_request_that_sat_out_and_of_a_row_used_again(geponex_folders, dtype):
    """The row of the token before lives in the request's state: a request that leaves a row behind must not hand its last
    token to the next request in that row (whose first token is shifted towards zeros)."""
    folder = geponex_folders("dense_alone")
    a, b = cases.prompts_for("dense_alone", lengths=[9, 6])
    runner = cases.runner_for(folder, DEV, dtype, num_pages=2, max_requests=1)
    for ids in (a, b, a):
        row = runner.admit()
        got = cases.step_all(runner, row, ids, [4, 1, 2])
        runner.release(row)
        ref = _logits(folder, ids)
        assert float((got - ref).abs().max()) <= cases.tol(dtype, ref, alone=True)
    # the first token's logits do depend on what stands before it, so a stale row would show
    ref = _logits(folder, [a[-1]] + b)
    assert float((ref[1] - _logits(folder, b)[0]).abs().max()) > 3 * cases.tol(dtype, ref, alone=True)


@pytest.mark.parametrize("dtype", DTYPES)
def test_first_tokens_and_long_decoding(geponex_folders, dtype):
    """A request of one token, then 150 tokens decoded one by one (through the captured graphs of single-token steps, over
    page borders), beside a second request that joins and leaves."""
    from vt_transformer_b200.engine.batch import StepEntry
    folder = geponex_folders(cases.for_dtype("mix", dtype))
    a, b = cases.prompts_for("mix", seed=9, lengths=[151, 40])
    runner = cases.runner_for(folder, DEV, dtype, num_pages=14, max_requests=2)
    ra = runner.admit()
    got_a, got_b, rb = [], [], None
    for i, tok in enumerate(a):
        entries = [StepEntry(ra, [tok], [0])]
        if 30 <= i < 30 + len(b):
            if rb is None:
                rb = runner.admit()
            entries.append(StepEntry(rb, [b[i - 30]], [0]))
        logits = runner.step(entries).double().cpu()
        got_a.append(logits[0])
        if len(entries) == 2:
            got_b.append(logits[1])
            if i - 30 == len(b) - 1:
                runner.release(rb)
    runner.check_status()
    for got, ids in ((got_a, a), (got_b, b)):
        cases.within(torch.stack(got), folder, ids, dtype)
    assert runner._graphs, "single-token steps did not run as captured graphs"


# ----------------------------------------------------------------------------- the entry point


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["mix", "wide"])
def test_greedy_generation_through_the_entry_point(geponex_folders, name, dtype):
    cases.greedy_generation(geponex_folders(cases.for_dtype(name, dtype)), name, DEV, dtype)


def test_trace_replay_command(geponex_folders, tmp_path):
    folder = geponex_folders("mix")
    prompts = cases.prompts_for("mix")
    trace = helpers.trace_mixed(prompts, max_live=4, seed=2)
    got = helpers.run_trace_cli(folder, trace, "float32", str(tmp_path / "out"), helpers.tokens_needed(trace, 64))
    cases.compare(folder, prompts, trace, got, "float32")


def test_generate_from_the_command_line_greedy(geponex_folders):
    import os
    import subprocess
    import sys
    folder = geponex_folders("wide")
    prompts = cases.prompts_for("wide")[:2]
    base = [sys.executable, "-m", "vt_transformer_b200", "generate", "--model", folder, "--dtype", "float32", "--max-tokens", "6",
            "--ignore-eos", "--num-pages", "16", "--max-seq-len", "128", "--page-size", "16", "--temperature", "0"]
    for p in prompts:
        base += ["--prompt-ids", ",".join(str(t) for t in p)]
    res = subprocess.run(base, capture_output=True, text=True, timeout=600, env=dict(os.environ, PYTHONPATH=helpers.ROOT), cwd=helpers.ROOT)
    assert res.returncode == 0, res.stderr[-3000:]
    lines = [[int(t) for t in l.split()] for l in res.stdout.splitlines() if l.strip()]
    assert len(lines) == 2 and all(len(l) == 6 for l in lines)
    for p, o in zip(prompts, lines):
        ref = _logits(folder, list(p) + o)
        for i, tok in enumerate(o):
            row = ref[len(p) - 1 + i]
            assert float(row.max() - row[tok]) <= 2 * cases.tol("float32", ref)
