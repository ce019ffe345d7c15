"""The kernels as Python functions over torch tensors.

Every function runs a hand-written sm_100a kernel of ``csrc``; the matrix products too (the
reference's engine calls cuBLASLt for them, v1/tensortype/cuda_kernels/lt_sgemm.cu:55-126; here
they are tcgen05 kernels of the package, and an FFMA kernel in 32-bit).  There is no CPU path and
no fallback: if the extension cannot be loaded or built, the first call raises.

``backend()`` returns the extension module.  Tests of the host-side logic may put an
object with the same functions in its place (``use_backend``); nothing in the package
does.
"""
from __future__ import annotations

import os
from typing import Optional

import torch

_backend = None
launches = 0          # kernels of this package enqueued so far (one for each call below)


def backend():
    global _backend
    if _backend is None:
        if not torch.cuda.is_available():
            raise RuntimeError("vt_transformer_b200 runs on a CUDA device (B200, sm_100a) only; "
                               "torch.cuda.is_available() is False and there is no CPU path")
        from ..csrc import build
        _backend = build.load()
    return _backend


def use_backend(obj) -> None:
    """Replaces the kernel module (for tests of the host-side logic).  ``None`` restores
    the real one at the next call."""
    global _backend
    _backend = obj


# --------------------------------------------------------------------------- elementwise


def embedding(table: torch.Tensor, ids: torch.Tensor, out: torch.Tensor, status=None, scale: float = 1.0) -> torch.Tensor:
    """out[t] = scale * table[ids[t]] as float32 rows (id -1: a row of zeros)."""
    backend().embedding(table, ids, out, status, float(scale))
    return out


def logits_scale_cap(logits: torch.Tensor, scale: float = 1.0, cap: float = 0.0) -> torch.Tensor:
    """logits = cap * tanh(scale * logits / cap) in place, in 32-bit; cap 0 applies the scale alone."""
    backend().logits_scale_cap(logits, float(scale), float(cap))
    return logits


class SplitSum:
    """The result [T, N] of a matrix product as the unadded 32-bit shares [shares, T, N] that the CTAs working
    on different parts of the inner dimension have left (``linear_to_stream``).  ``rmsnorm`` takes it as its
    delta and adds the shares, in the order of their index, while it reads them: the product's kernel is spared
    the merge of the shares at its end, and the delta reaches the 32-bit residual stream unrounded."""

    def __init__(self, shares: torch.Tensor):
        self.shares = shares

    @property
    def shape(self):
        return self.shares.shape[1:]

    @property
    def device(self):
        return self.shares.device

    def dense(self, dtype=None) -> torch.Tensor:
        """The sum as an ordinary tensor (tests, and parts that need one)."""
        total = self.shares[0].clone()
        for i in range(1, self.shares.shape[0]):
            total += self.shares[i]
        return total if dtype is None else total.to(dtype)


def dense(t, dtype=None) -> torch.Tensor:
    """``t`` as an ordinary tensor, whether it is one or a ``SplitSum``."""
    if isinstance(t, SplitSum):
        return t.dense(dtype)
    return t if dtype is None else t.to(dtype)


def _post(post):
    """(weight, eps, mult) of a delta that is normed before it is added, as the kernels' last three arguments."""
    if post is None:
        return ()
    weight, eps, mult = post
    return (weight, float(eps), float(mult))


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float, out, delta=None,
            rows: Optional[torch.Tensor] = None, status=None, post=None, groups: int = 1, x_scale: float = 1.0,
            to_stream: bool = False) -> torch.Tensor:
    """out = weight * v * rsqrt(mean(v^2) + eps) over the rows ``rows`` (all) of v = x_scale * x + delta, which is
    written back to x.  ``delta``: None, a tensor of out's dtype, or a ``SplitSum``.  With ``post`` = (w [H] float32,
    e, m) the delta is normed and scaled first, all in 32-bit: v = x + m * w * delta * rsqrt(mean(delta^2) + e).
    ``groups``: a row is cut into that many equal consecutive parts and each is divided by its own root mean square.
    ``to_stream``: x takes the normed row (32-bit, unrounded) instead of the sum, for a layer whose norm comes after the
    sum; ``out`` may then be None where nothing reads the rounded copy."""
    if isinstance(delta, SplitSum):
        delta = delta.shares
    if post is not None and delta is None:
        raise ValueError("rmsnorm: a delta to norm before it is added was announced and none came")
    if groups == 1 and x_scale == 1.0 and not to_stream:
        backend().rmsnorm(x, delta, weight, float(eps), out, rows, status, *_post(post))
    else:
        weight_post = _post(post) if post is not None else (None, 0.0, 1.0)
        backend().rmsnorm(x, delta, weight, float(eps), out, rows, status, *weight_post, int(groups), float(x_scale), bool(to_stream))
    return out


def layernorm(x: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor, delta=None,
              rows: Optional[torch.Tensor] = None, status=None, post=None) -> torch.Tensor:
    """out = weight * (v - mean(v)) * rsqrt(var(v) + eps) over the rows ``rows`` (all) of v = x + delta, which is
    written back to x; var is the mean of the squared deviations.  ``delta`` and ``post`` as for ``rmsnorm``."""
    if isinstance(delta, SplitSum):
        delta = delta.shares
    if post is not None and delta is None:
        raise ValueError("layernorm: a delta to norm before it is added was announced and none came")
    backend().layernorm(x, delta, weight, float(eps), out, rows, status, *_post(post))
    return out


def polynorm(z: torch.Tensor, coefficients: torch.Tensor, eps: float, out: torch.Tensor, n_mean: int = 0) -> torch.Tensor:
    """out = a N(z) + b N(z^2) + c N(z^3) + e row by row, N(y) = y / sqrt(mean(y^2) + eps), (a, b, c, e) the four
    float32 numbers of ``coefficients``; powers and means in 32-bit.  ``out`` may be ``z``.  With ``n_mean`` the means
    are over the first n_mean columns (the others are zero padding of a product whose matrix was padded)."""
    backend().polynorm(z, coefficients, float(eps), out, int(n_mean))
    return out


def head_norm_gate(o: torch.Tensor, y: torch.Tensor, gate_col: int, weight: torch.Tensor, weight_per_channel: bool,
                   eps: float, act: str, out: torch.Tensor, out_col: int, out_scale: float, heads: int, v_dim: int,
                   token_seq: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[t, out_col + h * v_dim + i] = out_scale * o[t, h, i] / sqrt(mean_i(o[t, h, :]^2) + eps) * w * act(gate)
    for the 32-bit o [T, heads * v_dim] of a recurrent mixer; gate = y[t, gate_col + h * v_dim + i]; w = weight[i]
    (a weight [v_dim] shared by the heads) or, with ``weight_per_channel``, weight[h * v_dim + i]; ``act`` is
    "silu" or "sigmoid".  32-bit until the one rounding into ``out``.  With ``token_seq`` (the step's sequence index
    of every token) the rows of padding tokens (-1), for which nothing ran, become zero."""
    backend().head_norm_gate(o, y, int(gate_col), weight, bool(weight_per_channel), float(eps), _GATE_ACTS[act], out,
                             int(out_col), float(out_scale), int(heads), int(v_dim), token_seq)
    return out


_GATE_ACTS = {"silu": 0, "sigmoid": 1}


# Threads of a scan kernel's CTA in a step whose sequences bring 16 tokens and more on average (portions of prompts):
# a head's column blocks then spread over several SMs.  Steps of single tokens keep a head in one CTA (0: the kernel's own
# bound).  Measured on a B200 at widths 1,024 and 4,096: a prompt of 4,096 tokens 1.4 to 1.8 times faster with 256 than
# with the kernel's 1,024; a decode step of 64 requests 1.3 to 1.5 times slower.
SCAN_WALK_THREADS = int(os.environ.get("VTB200_SCAN_WALK_THREADS", "256"))


def _scan_threads(ctx) -> int:
    return SCAN_WALK_THREADS if ctx.n_tokens >= 16 * max(1, ctx.n_seqs) else 0


def gla_scan(y, q_col: int, k_col: int, v_col: int, a_col: int, a2: torch.Tensor, a2_bias: torch.Tensor, inv_tau: float,
             q_scale: float, state: torch.Tensor, ctx, o: torch.Tensor, heads: int, dim: int, v_dim: int, status=None):
    """Gated linear attention over the step's tokens, sequence by sequence and head by head, in the order of the
    tokens: S <- diag(alpha_t) S + k_t v_t^T, o_t = S^T (q_scale * q_t), with log alpha = log sigmoid(z) * inv_tau and
    z = a2 (low-rank input at ``a_col``) + a2_bias.  q, k, v and the low-rank input are columns of ``y``; ``state``
    [request rows, heads, dim, v_dim] (float32) is read at the step's ``ctx.rows`` and left as after the last token;
    ``o`` [T, heads * v_dim] is float32.  Decay, state and sums are 32-bit."""
    backend().gla_scan(y, int(q_col), int(k_col), int(v_col), int(a_col), a2, a2_bias, float(inv_tau), float(q_scale),
                       state, ctx.cu_q, ctx.rows, o, int(heads), int(dim), int(v_dim), status, _scan_threads(ctx))
    return o


def delta_scan(y, r_col: int, k_col: int, v_col: int, a_col: int, w1_col: int, w2: torch.Tensor, w0: torch.Tensor,
               a_bias: torch.Tensor, decay_rate: float, key_eps: float, state: torch.Tensor, ctx, o: torch.Tensor,
               heads: int, dim: int, status=None):
    """The generalized delta rule over the step's tokens, sequence by sequence and head by head:
    S <- diag(w_t) S - (a_t * u_t)(u_t^T S) + k_t v_t^T, o_t = S^T r_t, with u = k / sqrt(sum(k^2) + key_eps),
    w = exp(-decay_rate * sigmoid(w2 tanh(low-rank input at ``w1_col``) + w0)) and a = sigmoid(y at ``a_col`` + a_bias).
    ``state`` [request rows, heads, dim, dim] float32; ``o`` [T, heads * dim] float32."""
    backend().delta_scan(y, int(r_col), int(k_col), int(v_col), int(a_col), int(w1_col), w2, w0, a_bias, float(decay_rate),
                         float(key_eps), state, ctx.cu_q, ctx.rows, o, int(heads), int(dim), status, _scan_threads(ctx))
    return o


# A sequence that brings this many tokens in a step, twice over, has its retention walk cut into up to RETENTION_SEGMENTS
# segments that run side by side (see ``retention_scan``).
RETENTION_SEGMENT_MIN = int(os.environ.get("VTB200_RETENTION_SEGMENT_MIN", "128"))
RETENTION_SEGMENTS = int(os.environ.get("VTB200_RETENTION_SEGMENTS", "8"))


class _RetentionPlan:
    """How a step's long walks are cut: the segments as the scan kernel's sequences (``cu``, ``rows``: a request's row
    for a sequence's first segment, -(n + 1) for its later segment n), for every cut sequence its row, its first later
    segment and their count, every later segment's length, and the tiles of up to 32 tokens of the later segments."""

    def __init__(self, ctx, device):
        import numpy as np
        cu, rows, seq_row, seq_first, seq_count, seg_len, tiles = [], [], [], [], [], [], []
        for s in ctx.seqs:
            pieces = min(RETENTION_SEGMENTS, s.length // max(1, RETENTION_SEGMENT_MIN))
            if pieces < 2:
                cu.append(s.offset)
                rows.append(s.row)
                continue
            size = -(-s.length // pieces)
            seq_row.append(s.row)
            seq_first.append(len(seg_len))
            for a in range(0, s.length, size):
                b = min(s.length, a + size)
                cu.append(s.offset + a)
                if a == 0:
                    rows.append(s.row)
                    continue
                rows.append(-(len(seg_len) + 1))
                tiles += [(len(seg_len), s.offset + t, min(32, b - t), s.offset + a) for t in range(a, b, 32)]
                seg_len.append(b - a)
            seq_count.append(len(seg_len) - seq_first[-1])
        cu.append(ctx.n_tokens)
        self.n_later = len(seg_len)
        if not self.n_later:
            return
        parts = [cu, rows, seq_row, seq_first, seq_count, seg_len, [v for t in tiles for v in t]]
        offs, total = [], 0
        for p in parts:
            offs.append(total)
            total += (len(p) + 3) & ~3                       # every array starts on a 16-byte boundary
        host = torch.zeros(total, dtype=torch.int32)
        for o, p in zip(offs, parts):
            host[o:o + len(p)] = torch.from_numpy(np.asarray(p, dtype=np.int32))
        if torch.device(device).type == "cuda":
            host = host.pin_memory()
        buf = host.to(device, non_blocking=True)
        seg = lambda i: buf[offs[i]:offs[i] + len(parts[i])]
        self.cu, self.rows, self.seq_row, self.seq_first, self.seq_count, self.seg_len = (seg(i) for i in range(6))
        self.tiles = seg(6).view(-1, 4)
        self.n_segments = len(rows)


def retention_scan(y, q_col: int, k_col: int, v_col: int, decay: torch.Tensor, k_scale: float, frequencies, state: torch.Tensor,
                   ctx, o: torch.Tensor, heads: int, dim: int, v_dim: int, status=None, act: bool = False):
    """Retention over the step's tokens, sequence by sequence and head by head, in the order of the tokens:
    S <- decay[h] S + (k_scale * k_t) v_t^T, o_t = S^T q_t, after the first 2 * len(frequencies) dimensions of every
    head of q and k were rotated, pairs (i, i + len), by position * frequencies[i] (a 32-bit product, in 32-bit;
    ``frequencies`` None: no rotation).  q, k and v are columns of ``y``; ``decay`` [heads] float32; ``state``
    [request rows, heads, dim, v_dim] (float32) is read at the step's ``ctx.rows`` and left as after the last token;
    ``o`` [T, heads * v_dim] is float32.  Rotation, state and sums are 32-bit.

    A sequence that brings many tokens is cut into segments that run side by side: the recurrence is linear in the
    state it starts from, so the later segments start from zeros, one kernel carries the state from segment to segment,
    and one adds decay^(t - t0 + 1) S_before^T q_t to the later segments' tokens; 32-bit throughout, only the order of
    the sums differs.  ``act``: q, k and v pass through silu (z / (1 + exp(-z)), 32-bit) as they are read."""
    be = backend()
    act = 1 if act else 0
    plan = None
    if ctx.seqs and ctx.max_q_len >= 2 * RETENTION_SEGMENT_MIN and RETENTION_SEGMENTS > 1:
        key = ("retention_plan", RETENTION_SEGMENT_MIN, RETENTION_SEGMENTS)
        plan = ctx.extras.get(key)
        if plan is None:
            plan = ctx.extras[key] = _RetentionPlan(ctx, y.device)
    if plan is None or not plan.n_later:
        be.retention_scan(y, int(q_col), int(k_col), int(v_col), decay, float(k_scale), frequencies, ctx.positions, state,
                          ctx.cu_q, ctx.rows, o, int(heads), int(dim), int(v_dim), status, _scan_threads(ctx), None, act)
        return o
    ends = torch.empty((plan.n_later, heads, dim, v_dim), dtype=torch.float32, device=y.device)
    starts = torch.empty_like(ends)
    threads = SCAN_WALK_THREADS if ctx.n_tokens >= 16 * plan.n_segments else 0
    be.retention_scan(y, int(q_col), int(k_col), int(v_col), decay, float(k_scale), frequencies, ctx.positions, state, plan.cu,
                      plan.rows, o, int(heads), int(dim), int(v_dim), status, threads, ends, act)
    global launches
    launches += 2
    be.retention_carry(state, ends, starts, plan.seq_row, plan.seq_first, plan.seq_count, plan.seg_len, decay, status)
    be.retention_fix(y, int(q_col), ctx.positions, frequencies, starts, plan.tiles, decay, o, act)
    return o


def attention_prepare(y, q_col: int, k_col: int, v_col: int, ctx, frequencies, norm_eps, k_cache, v_cache, block_table,
                      heads: int, kv_heads: int, dim: int, v_dim: int, store: bool = True, status=None, v_heads=None,
                      q_weight=None, k_weight=None, norm_first: bool = False, whole_projection: bool = False,
                      rot_mult: float = 1.0, q_temp=None) -> None:
    """What the general attention does to a step's q, k and v (columns of ``y``) before its keys are walked: the
    first 2 * len(frequencies) dimensions of every head of q and k are rotated, pairs (i, i + len), by
    position * frequencies[i] (a 32-bit product; ``frequencies`` None: no rotation); with ``norm_eps`` not None,
    every head of q and k is divided by sqrt(mean(.^2) + norm_eps) and multiplied by ``q_weight`` / ``k_weight``
    ([dim] float32, or None), after the rotation or, with ``norm_first``, before it; q is written back into ``y``, k and
    v go into their pages ([pages, kv_heads, page_size, dim] and [pages, v_heads, page_size, v_dim]; ``v_heads``
    None: as many as kv_heads) if ``store``.  ``whole_projection`` (with ``norm_first``): the mean square is taken over all
    heads of q together (and of k) and the weights are [heads * dim] and [kv_heads * dim].  ``rot_mult`` multiplies cos and
    sin.  ``q_temp`` = (c, n): q is multiplied by 1 + c ln(floor((position + 1) / n) + 1), last of all."""
    args = (y, int(q_col), int(k_col), int(v_col), ctx.positions, ctx.token_seq, frequencies,
            -1.0 if norm_eps is None else float(norm_eps), k_cache, v_cache, block_table, int(heads),
            int(kv_heads), int(dim), int(v_dim), bool(store), status,
            int(kv_heads if v_heads is None else v_heads), q_weight, k_weight, bool(norm_first))
    if whole_projection or rot_mult != 1.0 or q_temp is not None:
        coef, every = (float(q_temp[0]), int(q_temp[1])) if q_temp is not None else (0.0, 1)
        backend().attention_prepare(*args, bool(whole_projection), float(rot_mult), coef, every)
    else:
        backend().attention_prepare(*args)


def attention_general(y, q_col: int, out, out_col: int, out_scale: float, k_cache, v_cache, ctx, block_table, heads: int,
                      kv_heads: int, dim: int, v_dim: int, window, chunk, scale: float, status=None, keep_first: int = 0,
                      maps: int = 1, lam: float = 0.0, sub_eps: float = 0.0, sinks=None, values_in_keys: bool = False,
                      softcap=None, gate: str = "none", gate_col: int = 0):
    """out[t, out_col + h * v_dim + :] = out_scale * softmax(scale * q . k_j) v_j over the keys j that token t at
    position p sees: j <= p, and j > p - window or j < keep_first (if a window is given), and j // chunk == p // chunk
    (if chunks are).  q is read at column ``q_col`` of ``y``; keys of size ``dim`` and values of size ``v_dim`` from
    their pages.  ``maps`` 2: every head has two queries [2, dim] and every head of values two heads of keys (k pages
    [pages, kv_heads * 2, page_size, dim]); with a_1 and a_2 the two attentions over the same values,
    o = a_1 - lam * a_2 and out = out_scale * o / sqrt(mean(o^2) + sub_eps), all in 32-bit.
    ``sinks`` [heads] float32: one more term exp(sinks[h]) in the softmax's denominator, without a key or a value and not
    scaled.  ``values_in_keys``: a value is the first ``v_dim`` numbers of its key's row (``v_cache`` is ``k_cache``).
    ``softcap`` c: a score becomes c tanh(score / c) after the scale.  ``gate`` "head": head h's result is multiplied by
    sigmoid(y[t, gate_col + h]); "element": element i of it by sigmoid(y[t, gate_col + h * v_dim + i])."""
    args = (y, int(q_col), out, int(out_col), float(out_scale), k_cache, v_cache, ctx.positions,
            ctx.token_seq, block_table, int(heads), int(kv_heads), int(dim), int(v_dim),
            int(window) if window else 0, int(chunk) if chunk else 0, float(scale), status,
            int(keep_first), int(maps), float(lam), float(sub_eps), sinks, bool(values_in_keys))
    if softcap or gate != "none":
        backend().attention_general(*args, float(softcap) if softcap else 0.0, _ATTENTION_GATES[gate], int(gate_col))
    else:
        backend().attention_general(*args)
    return out


_ATTENTION_GATES = {"none": 0, "head": 1, "element": 2}


def gated_delta_scan(y, q_col: int, k_col: int, v_col: int, b_col: int, a_col: int, conv_q, conv_k, conv_v, a_log: torch.Tensor,
                     dt_bias: torch.Tensor, key_eps: float, q_scale: float, state: torch.Tensor, tail, ctx, o: torch.Tensor,
                     heads: int, kv_heads: int, dim: int, v_dim: int, status=None):
    """The delta rule with one decay a head over the step's tokens, sequence by sequence and head by head, in the order of
    the tokens.  q and k ([kv_heads * dim]) and v ([heads * v_dim]) are columns of ``y``; each passes a causal convolution
    over time, channel by channel (``conv_q``, ``conv_k``, ``conv_v``: float32 [channels, taps], the last tap the present
    token's; None: no convolution), whose inputs before the step's first token come from ``tail`` [request rows, taps - 1,
    channels of q + k + v] (float32, oldest first; this kernel reads it, ``conv_tail_update`` renews it), and silu; q and k
    are divided, head by head, by sqrt(sum(.^2) + key_eps), q multiplied by ``q_scale``.  beta = sigmoid(y at ``b_col`` + h),
    g = exp(-exp(a_log[h]) softplus(y at ``a_col`` + h + dt_bias[h])).  S <- g S; u = beta (v - S^T k); S <- S + k u^T;
    o = S^T q, head h with q/k head h // (heads / kv_heads).  ``state`` [request rows, heads, dim, v_dim] float32 is read at
    the step's ``ctx.rows`` and left as after the last token; ``o`` [T, heads * v_dim] float32.  All in 32-bit."""
    backend().gated_delta_scan(y, int(q_col), int(k_col), int(v_col), int(b_col), int(a_col), conv_q, conv_k, conv_v, a_log, dt_bias,
                               float(key_eps), float(q_scale), state, tail, ctx.cu_q, ctx.rows, o, int(heads), int(kv_heads),
                               int(dim), int(v_dim), status, _scan_threads(ctx))
    return o


def conv_tail_update(y, cols, widths, tail: torch.Tensor, ctx, status=None) -> None:
    """Renews what a short convolution keeps of a request: ``tail`` [request rows, n, channels] (float32) holds the last n
    inputs of every channel, oldest first; the channels are the columns [cols[i], cols[i] + widths[i]) of ``y`` one group
    after the other.  After the step it holds the last n inputs again: the step's last tokens, and before them what it held."""
    backend().conv_tail_update(y, [int(c) for c in cols], [int(w) for w in widths], tail, ctx.cu_q, ctx.rows, status)


def memory_scan(y, q_col: int, k_col: int, v_col: int, i_col: int, f_col: int, i_bias: torch.Tensor, f_bias: torch.Tensor,
                gate_cap: float, q_scale: float, den_eps: float, state: torch.Tensor, ctx, o: torch.Tensor, heads: int, dim: int,
                v_dim: int, status=None):
    """A matrix of memory a head with exponential gates over the step's tokens, in their order.  q, k ([heads * dim]) and v
    ([heads * v_dim]) are columns of ``y``; i = c tanh((y at ``i_col`` + h + i_bias[h]) / c) and
    f = log sigmoid(c tanh((y at ``f_col`` + h + f_bias[h]) / c)), c = ``gate_cap``.  m' = max(f + m, i);
    S <- exp(f + m - m') S + exp(i - m') k v^T; n likewise with k alone; o = S^T (q_scale q) / (max(|n . q_scale q|, exp(-m')) + den_eps).
    ``state`` [request rows, heads, dim + 1, v_dim + 1] float32: S in [:dim, :v_dim], n in [:dim, v_dim], m at [dim, 0].
    ``o`` [T, heads * v_dim] float32.  All in 32-bit."""
    backend().memory_scan(y, int(q_col), int(k_col), int(v_col), int(i_col), int(f_col), i_bias, f_bias, float(gate_cap),
                          float(q_scale), float(den_eps), state, ctx.cu_q, ctx.rows, o, int(heads), int(dim), int(v_dim), status,
                          _scan_threads(ctx))
    return o


def normed_sum(parts, weights, eps: float, scales, out: torch.Tensor) -> torch.Tensor:
    """out = sum_i scales[i] * weights[i] * parts[i] / sqrt(mean(parts[i]^2) + eps), row by row, for float32 parts [T, H]
    (up to four) and weights [H]; all in 32-bit, the sum in the order of i."""
    backend().normed_sum(list(parts), list(weights), float(eps), [float(c) for c in scales], out)
    return out


def add_rows(x: torch.Tensor, other: torch.Tensor) -> torch.Tensor:
    """x += other for float32 [T, H] (the residual stream and another stream of its shape)."""
    backend().add_rows(x, other)
    return x


# Picks (tokens of a step times the experts each uses) from which a mixture of experts groups its tokens by expert
# instead of running every expert on every token.  Below it, and in every step of single tokens, the two packed
# products read each expert's weights once, which a small batch does anyway, and the step stays a CUDA graph.
EXPERTS_GROUPED_MIN_PICKS = int(os.environ.get("VTB200_EXPERTS_GROUPED_MIN_PICKS", "1024"))


_ROUTER_WEIGHTS = {"softmax": 0, "sigmoid_share": 1}


def route_topk(logits, top: int, ids: torch.Tensor, weights: torch.Tensor, x=None, router=None, weights_by: str = "softmax",
               scale: float = 1.0) -> None:
    """ids[t, k] and weights[t, k]: the ``top`` largest router logits of every token in falling order (the lower index
    among equals) and the softmax over them.  ``logits`` [tokens, experts] float32, or None with the tokens' input rows
    ``x`` [tokens, width] and the router's matrix ``router`` [experts, width] (float32), from which the kernel forms
    them as 32-bit dot products.  ``weights_by`` "sigmoid_share": a pick weighs as sigmoid(logit) over the picks' sum of
    them (+ 1e-20), times ``scale``."""
    backend().route_topk(logits, int(top), ids, weights, x, router, _ROUTER_WEIGHTS[weights_by], float(scale))


def expert_lists(ids: torch.Tensor, lists: torch.Tensor, counts: torch.Tensor) -> None:
    """lists[e, :counts[e]]: the picks (flat index t * top + k of ``ids``) that chose expert e, in rising order."""
    backend().expert_lists(ids, lists, counts)


def gather_picks(x: torch.Tensor, lists: torch.Tensor, counts: torch.Tensor, top: int, rows: torch.Tensor, where: torch.Tensor) -> None:
    """rows: the rows of x sorted by expert (expert 0's picks in the order of its list, then expert 1's, ...), row of pick
    p being x[p // top]; where[p]: the row at which pick p lies."""
    backend().gather_picks(x, lists, counts, int(top), rows, where)


def combine_picks(y: torch.Tensor, where: torch.Tensor, weights: torch.Tensor, shared_y, out: torch.Tensor) -> torch.Tensor:
    """out[t] = sum_k weights[t, k] * y[where[t * top + k]] (+ shared_y[t]), in 32-bit in the order of k, one rounding."""
    backend().combine_picks(y, where, weights, shared_y, out)
    return out


def attention_differential(y, q_col: int, out, out_col: int, out_scale: float, k_cache, v_cache, ctx, block_table, heads: int,
                           kv_heads: int, dim: int, v_dim: int, window, keep_first: int, scale: float, lam: float, sub_eps: float,
                           status=None):
    """Differential attention of the step's tokens over the paged keys and values of their sequences: every head has
    two queries [2, dim] (at column ``q_col`` of ``y``) and every head of values two heads of keys; with a_1, a_2 the two
    softmax attentions over the same values, out[t, out_col + h * v_dim + :] = out_scale * o / sqrt(mean(o^2) + sub_eps),
    o = a_1 - lam * a_2.  Position p sees j <= p with p - j < window or j < keep_first.  bfloat16 at the sizes the
    tensor-core kernel takes runs that kernel (prompt portions in tiles of 64 rows of (token, head of the group);
    single tokens a CTA for each (sequence, head of values)); everything else, and all of float32, the plain kernel."""
    be = backend()
    if (y.dtype == torch.bfloat16 and ATTENTION_KERNEL in ("auto", "mma") and k_cache.shape[2] % 16 == 0 and q_col % 8 == 0
            and out_col % 8 == 0 and be.attention_diff_supports(int(dim), int(v_dim), int(heads), int(kv_heads))):
        singles = ctx.max_q_len == 1 and ctx.n_tokens == ctx.n_seqs
        tiles = None if singles else _attention_tiles(ctx, be.attention_diff_tile_rows() // (heads // kv_heads), y.device)
        be.attention_diff(y, int(q_col), out, int(out_col), float(out_scale), k_cache, v_cache, ctx.cu_q, ctx.q_start, block_table,
                          tiles, int(heads), int(kv_heads), int(dim), int(v_dim), int(window) if window else 0, int(keep_first),
                          float(scale), float(lam), float(sub_eps), status)
        return out
    return attention_general.__wrapped__(y, q_col, out, out_col, out_scale, k_cache, v_cache, ctx, block_table, heads, kv_heads, dim,
                                         v_dim, window, None, scale, status=status, keep_first=keep_first, maps=2, lam=lam,
                                         sub_eps=sub_eps)


LATENT_TARGET_CTAS = 296     # CTAs that the latent attention of a step of single tokens aims at (two for each SM)
LATENT_MAX_RUNS = 16         # the most runs of keys that a sequence is cut into for that (the merge kernel's limit)


def attention_latent(q, q_col: int, out, out_col: int, pages, ctx, block_table, heads: int, key: int, v_dim: int, scale: float,
                     sinks=None, status=None):
    """Softmax attention of the step's tokens over paged rows that all heads share: head h's query [key] stands at
    q[t, q_col + h * key + :], a cached token's row of ``pages`` [pages, 1, page_size, key] is every head's key and its first
    ``v_dim`` numbers every head's value; out[t, out_col + h * v_dim + :] = sum_j p_j row_j[:v_dim] with
    p = softmax_j(scale q . row_j) over the keys j up to the token's position.  ``sinks`` [heads] float32: exp(sinks[h])
    joins the denominator (no key, no value, not scaled).  bfloat16 at the sizes the tensor-core kernel takes runs that
    kernel (tiles of 64 rows of (token, head) that share each block of keys; a single token's tile holds its heads, and in a
    step of single tokens every sequence's keys are cut into runs with a CTA each, merged in the order of the runs);
    everything else, and all of float32, the plain kernel."""
    be = backend()
    if (q.dtype == torch.bfloat16 and ATTENTION_KERNEL in ("auto", "mma") and q_col % 8 == 0 and out_col % 2 == 0
            and be.attention_latent_supports(int(key), int(v_dim))):
        singles = ctx.max_q_len == 1 and ctx.n_tokens == ctx.n_seqs
        rows = be.attention_latent_tile_rows()
        tiles = None if singles else _attention_tiles(ctx, rows // min(int(heads), rows), q.device)
        part = None
        if singles:
            # few sequences leave most SMs without a CTA: every sequence's keys are cut into runs, a CTA each
            ctas = ctx.n_seqs * -(-int(heads) // rows)
            runs = min(LATENT_MAX_RUNS, max(1, LATENT_TARGET_CTAS // ctas))
            if runs > 1:
                part = torch.empty((runs, q.shape[0], int(heads), int(v_dim) + 2), dtype=torch.float32, device=q.device)
        be.attention_latent(q, int(q_col), out, int(out_col), pages, ctx.cu_q, ctx.q_start, block_table, tiles, int(heads), int(key),
                            int(v_dim), float(scale), sinks, part)
        return out
    return attention_general.__wrapped__(q, q_col, out, out_col, 1.0, pages, pages, ctx, block_table, heads, 1, key, v_dim, None, None,
                                         scale, status=status, sinks=sinks, values_in_keys=True)


def route_experts(logits, top: int, act: torch.Tensor, inter: int, x=None, router=None, weights_by: str = "softmax",
                  scale: float = 1.0) -> torch.Tensor:
    """For every token (row): the ``top`` largest of its router logits [experts] (float32; the lower index among
    equals) choose its experts, the softmax over the chosen logits weighs them; columns [e * inter, (e + 1) * inter) of
    ``act`` (what expert e's last product multiplies) are multiplied by expert e's weight, and set to zero for an
    expert that was not chosen.  Columns beyond experts * inter (an expert that every token uses) stay.  ``logits`` may be
    None with ``x`` and ``router`` given, and ``weights_by`` and ``scale``, as for ``route_topk``."""
    backend().route_experts(logits, int(top), act, int(inter), x, router, _ROUTER_WEIGHTS[weights_by], float(scale))
    return act


def token_shift(x: torch.Tensor, mu: torch.Tensor, state: torch.Tensor, ctx, out: torch.Tensor, status=None) -> torch.Tensor:
    """out[t] = x[t] + (x[t - 1] - x[t]) * mu for the 32-bit rows x [T, width], mu [width] float32; the row before a
    sequence's first token of the step is state[ctx.rows[seq]] (float32 [request rows, width], zeros at admission), which
    then takes the sequence's last row of the step.  Rows of padding tokens become zero."""
    backend().token_shift(x, mu, state, ctx.cu_q, ctx.rows, ctx.token_seq, out, status)
    return out


def latent_prepare(y, q_col: int, q_rank: int, kv_col: int, kv_rank: int, rot_dim: int, q_weight, k_weight, eps: float,
                   frequencies, mult: float, ctx, block_table, cq, pages, store: bool = True, status=None) -> None:
    """The two latents of every token, from the columns of ``y``: [q_col, q_col + q_rank) divided by its root mean square
    and multiplied by ``q_weight`` goes to cq[:, :q_rank]; [kv_col, kv_col + kv_rank) the same with ``k_weight``, and the
    ``rot_dim`` numbers behind it with their first 2 * len(frequencies) rotated (pairs (2i, 2i + 1), angle
    position * frequencies[i] as a 32-bit product, cos and sin times ``mult``; not normed), go side by side into the
    token's row of ``pages`` [pages, 1, page_size, kv_rank + rot_dim] if ``store``.  Norms and rotation in 32-bit."""
    backend().latent_prepare(y, int(q_col), int(q_rank), int(kv_col), int(kv_rank), int(rot_dim), q_weight, k_weight, float(eps),
                             frequencies, float(mult), ctx.positions, ctx.token_seq, block_table, cq, pages, bool(store), status)


def head_matmul(x, x_col: int, x_head: int, m, out, out_col: int, out_head: int, mode: str = "plain", tail: int = 0,
                frequencies=None, mult: float = 1.0, ctx=None, gate=None, gate_col: int = 0):
    """out[t, out_col + h * out_head + j] = sum_i x[t, x_col + h * x_head + i] * m[h, i, j] for m [heads, inner, outer], the
    sums in 32-bit in the order of i.  ``mode`` "rotated_tail": the ``tail`` numbers behind a head's inputs are rotated
    like ``latent_prepare``'s shared key part and copied behind the head's outputs; "gate": the result is multiplied by
    sigmoid(gate[t, gate_col + h * outer + j]) where ``gate`` is given."""
    code = {"plain": 0, "rotated_tail": 1, "gate": 2}[mode]
    backend().head_matmul(x, int(x_col), int(x_head), m, out, int(out_col), int(out_head), code, int(tail), frequencies,
                          float(mult), None if ctx is None else ctx.positions, None if ctx is None else ctx.token_seq, gate,
                          int(gate_col))
    return out


def xielu(z: torch.Tensor, out: torch.Tensor, a_pos: float, a_neg: float) -> torch.Tensor:
    """out = a_pos z^2 + z / 2 where z > 0, a_neg (exp(z) - 1 - z) + z / 2 elsewhere; 32-bit, one rounding."""
    backend().xielu(z, out, float(a_pos), float(a_neg))
    return out


def gate_clamp(gu: torch.Tensor, out: torch.Tensor, interleave: int, alpha: float, limit: float, split: int = 0,
               limit2: Optional[float] = None) -> torch.Tensor:
    """out = g sigmoid(alpha g) (u + 1) with g = min(gate, limit), u = clamp(up, -limit, limit); gu [T, 2 n] holds gate and
    up side by side or, with ``interleave`` 8, alternating in runs of 8.  Columns of out from ``split`` on take ``limit2``."""
    n = out.shape[1]
    backend().gate_clamp(gu, out, int(interleave), float(alpha), float(limit), int(split) if limit2 is not None else n,
                         float(limit if limit2 is None else limit2))
    return out


def scale_into(src: torch.Tensor, dst: torch.Tensor, dst_col: int, scale: float) -> torch.Tensor:
    """dst[:, dst_col : dst_col + n] = scale * src for src [T, n] (the product in 32-bit, one rounding)."""
    backend().scale_into(src, dst, int(dst_col), float(scale))
    return dst


def tensor_core_attention_takes(dtype, heads: int, kv_heads: int, head_dim: int, v_dim: int, page_size: int) -> bool:
    """Whether ``paged_attention`` runs bfloat16 tensor-core kernels at these sizes for every kind of step (values as
    wide as keys, a head size the kernels take, pages of a multiple of 16 tokens)."""
    return (dtype == torch.bfloat16 and v_dim == head_dim and page_size % 16 == 0 and ATTENTION_KERNEL in ("auto", "mma")
            and backend().attention_mma_supports(head_dim, heads, kv_heads, 1)
            and backend().attention_mma_supports(head_dim, heads, kv_heads, 4))


def silu_mul(gu: torch.Tensor, out: torch.Tensor, interleave: int = 0) -> torch.Tensor:
    """out = silu(gate) * up.  ``interleave`` 0: gu = [gate | up]; 8: gate and up columns alternate in
    runs of 8 (``interleave_gate_up``)."""
    backend().silu_mul(gu, out, interleave)
    return out


def interleave_gate_up(w_gate: torch.Tensor, w_up: torch.Tensor) -> torch.Tensor:
    """Packs the rows of the gate and up matrices [I, H] into one matrix [2 I, H] in runs of 8:
    g0..g7, u0..u7, g8..g15, u8..u15, ...  One product over it gives gate and up of the same 8
    features side by side, so that silu(gate) * up can be formed where the product's result lies
    (a thread's registers) and only [T, I] is written."""
    inter, hidden = w_gate.shape
    if inter % 8:
        raise ValueError(f"intermediate size {inter} must be a multiple of 8")
    return torch.stack([w_gate.view(inter // 8, 8, hidden), w_up.view(inter // 8, 8, hidden)], dim=1).reshape(
        2 * inter, hidden).contiguous()


# Bytes of the next product's weights that a weight-streaming product asks into L2 while it ends (0: none).
LOOK_AHEAD_BYTES = int(os.environ.get("VTB200_LOOK_AHEAD_BYTES", str(8 << 20)))
_PRODUCT_KINDS = {"linear": 0, "silu_mul": 1, "stream": 2}


def product_hint(w: torch.Tensor, kind: str):
    """What a part tells the product before one of its own: the matrix ``w`` [N, K] will be streamed next, by
    ``linear`` ("linear"), ``linear_silu_mul`` ("silu_mul") or ``linear_to_stream`` ("stream").  None for a
    matrix that the tcgen05 kernel does not take.  Passed as ``then=``; it changes no result."""
    if w is None or w.dtype != torch.bfloat16 or w.dim() != 2 or not w.is_cuda or not w.is_contiguous():
        return None
    return (w, _PRODUCT_KINDS[kind])


def _ahead(then) -> dict:
    if then is None or LOOK_AHEAD_BYTES <= 0:
        return {}
    return {"next_w": then[0], "next_epilogue": then[1], "next_bytes": LOOK_AHEAD_BYTES}


def linear_silu_mul(x: torch.Tensor, w_gate_up: torch.Tensor, out: torch.Tensor, status=None, then=None) -> torch.Tensor:
    """out[T, I] = silu(x Wg^T) * (x Wu^T) for ``w_gate_up = interleave_gate_up(Wg, Wu)``.  bfloat16: one
    tcgen05 kernel whose epilogue forms the product from the 32-bit sums.  Otherwise the product
    into [T, 2 I] and the elementwise kernel."""
    be = backend()
    if x.dtype == torch.bfloat16 and w_gate_up.dtype == torch.bfloat16 and FUSE_SILU and \
            not (x.shape[0] <= SKINNY_MAX_ROWS and SMALL_BATCH_KERNEL == "skinny"):
        scratch, counters = _split_workspace(x.device)
        global launches
        launches += 1
        be.gemm_tc(x, w_gate_up, None, out, status, scratch, counters, 1, **_ahead(then))
        return out
    gu = torch.empty((x.shape[0], w_gate_up.shape[0]), dtype=x.dtype, device=x.device)
    linear(x, w_gate_up, None, gu, status)
    be.silu_mul(gu, out, 8)
    return out


FUSE_SILU = True    # False: always the separate elementwise kernel (tests compare the two)


def rope_store(qkv, positions, cos_sin, k_cache, v_cache, token_seq, block_table, heads: int, kv_heads: int,
               head_dim: int, store: bool = True, status=None) -> None:
    backend().rope_store(qkv, positions, cos_sin, k_cache, v_cache, token_seq, block_table, heads, kv_heads,
                         head_dim, bool(store), status)


# --------------------------------------------------------------------------- matrix products


def linear(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor, status=None,
           then=None) -> torch.Tensor:
    """out[T, N] = x[T, K] w[N, K]^T (+ bias).  ``out`` is float32 or the dtype of x.  ``then``: the
    ``product_hint`` of the product that runs next, if the caller knows it.

    float32 x and w: the 32-bit kernel (FFMA in a fixed order, no TF32).  A weight kept in
    32-bit beside bfloat16 activations goes the same way, with x widened.  bfloat16: the
    tcgen05 kernel (TMA, tensor memory), with w as the 128-row operand for up to 256 rows of x
    and x beyond.
    """
    be = backend()
    if w.dtype == torch.float32:
        xf = x if x.dtype == torch.float32 else x.float()
        if out.dtype == torch.float32:
            be.gemm_simt(xf, w, bias, out)
        else:
            tmp = torch.empty(out.shape, dtype=torch.float32, device=out.device)
            be.gemm_simt(xf, w, bias, tmp)
            out.copy_(tmp)
        return out
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise TypeError(f"linear: unsupported dtypes x {x.dtype}, w {w.dtype}")
    m = x.shape[0]
    if m <= SKINNY_MAX_ROWS and SMALL_BATCH_KERNEL == "skinny":
        be.gemm_skinny(x, w, bias, out)
    else:
        scratch, counters = _split_workspace(x.device)
        be.gemm_tc(x, w, bias, out, status, scratch, counters, **_ahead(then))
    return out


STREAM_SHARES = os.environ.get("VTB200_STREAM_SHARES", "1") != "0"   # False: linear_to_stream always adds the shares itself


def linear_to_stream(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], status=None, then=None):
    """x w^T (+ bias) for a result that goes straight into the residual stream (``ResidualStream.add``): a
    tensor [T, N] of x's dtype, or, for bfloat16 batches small enough that the kernel cuts the inner dimension
    over CTAs, a ``SplitSum`` of the unadded 32-bit shares, which the next norm adds."""
    m = x.shape[0]
    # (a small matrix under a wide batch is faster with x as the 128-row operand and no shares: measured on a B200,
    # 256 rows by [1152, 896]: 21 us with shares, 15 us without; at 128 rows they are level)
    small_under_wide = m > 128 and w.shape[0] * w.shape[1] * 2 <= STREAM_SMALL_WEIGHT_BYTES
    if (STREAM_SHARES and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and 0 < m <= STREAM_MAX_ROWS
            and not small_under_wide and not (SMALL_BATCH_KERNEL == "skinny" and m <= SKINNY_MAX_ROWS)):
        be = backend()
        n, k = w.shape
        shares = torch.empty((be.gemm_tc_shares(m, n, k), m, n), dtype=torch.float32, device=x.device)
        global launches
        launches += 1
        be.gemm_tc(x, w, bias, shares, status, None, None, 2, **_ahead(then))
        return SplitSum(shares)
    out = torch.empty((m, w.shape[0]), dtype=x.dtype, device=x.device)
    return linear(x, w, bias, out, status, then)


_workspaces = {}


def _split_workspace(device):
    """Scratch and arrival counters with which the tcgen05 kernel cuts k over CTAs for small batches:
    8M floats and 4,096 counters a device, made once.  Launches that use them run in one stream."""
    ws = _workspaces.get(device)
    if ws is None:
        ws = (torch.empty(8 << 20, dtype=torch.float32, device=device), torch.zeros(4096, dtype=torch.int32, device=device))
        _workspaces[device] = ws
    return ws


SKINNY_MAX_ROWS = 64            # rows of x up to which the small-batch kernel may run
STREAM_MAX_ROWS = 256           # rows up to which w is the 128-row operand and products may leave their shares of k unadded
STREAM_SMALL_WEIGHT_BYTES = 8 << 20   # ... unless the matrix is this small and the batch has more than 128 rows
# "tc": the tcgen05 kernel with w as the 128-row operand; "skinny": mma.sync weight streaming.
# The environment variable VTB200_SMALL_BATCH_KERNEL overrides it (for measurements).
import os as _os
SMALL_BATCH_KERNEL = _os.environ.get("VTB200_SMALL_BATCH_KERNEL", "tc")
# "auto"; "mma": no tcgen05 attention (the mma.sync kernels only); "simt": the plain kernel (tests compare them)
ATTENTION_KERNEL = "auto"


# --------------------------------------------------------------------------- attention


def _attention_tiles(ctx, tokens_per_tile: int, device, first_seq: int = 0):
    """(sequence, first token) for every tile of the step: each sequence's new tokens in runs of
    ``tokens_per_tile``, ordered by falling number of keys; the sequences before ``first_seq`` are left out.
    Built once a step and kept in ``ctx.extras``."""
    key = ("attention_tiles", tokens_per_tile, first_seq)
    tiles = ctx.extras.get(key)
    if tiles is None:
        pairs = [(i, a) for i, s in enumerate(ctx.seqs) if i >= first_seq for a in range(0, s.length, tokens_per_tile)]
        # the tiles with the most keys first: the CTAs that start last are then the short ones
        pairs.sort(key=lambda p: -(ctx.seqs[p[0]].start + p[1]))
        host = torch.tensor(pairs, dtype=torch.int32).view(-1, 2)
        if torch.device(device).type == "cuda":
            host = host.pin_memory()
        tiles = host.to(device, non_blocking=True)
        ctx.extras[key] = tiles
    return tiles


MIXED_STEP_MIN_SINGLES = 2    # single tokens at the head of a mixed step from which they get a launch of their own


def _leading_single_tokens(ctx) -> int:
    """How many entries at the head of the step bring one token each (0 if all do: that is no mixed step)."""
    n = 0
    for s in ctx.seqs:
        if s.length != 1:
            break
        n += 1
    return n if n < len(ctx.seqs) else 0


def single_token_step_is_one_kernel(ctx, dtype, heads: int, kv_heads: int, head_dim: int) -> bool:
    """Whether ``rope_attention`` will run rotation, cache store and attention of this step as one kernel: a
    bfloat16 step of single tokens at sizes the tensor-core kernel takes.  That kernel also takes q, k and v as
    the unadded shares of the product before it (``linear_to_stream``)."""
    return (dtype == torch.bfloat16 and ATTENTION_KERNEL in ("auto", "mma") and FUSE_ROPE and ctx.max_q_len == 1
            and ctx.n_tokens == ctx.n_seqs and backend().attention_mma_supports(head_dim, heads, kv_heads, 1))


def rope_attention(qkv, out, cos_sin, k_cache, v_cache, ctx, block_table, heads: int, kv_heads: int, head_dim: int,
                   window: Optional[int], scale: float, store: bool = True, status=None) -> torch.Tensor:
    """Rotation of q and k by the tokens' positions, store of k and v into their pages (if ``store``),
    and attention over the pages: the three steps of the attention mixer between its two products.
    In a bfloat16 step of single tokens they are one kernel (the attention kernel rotates q in its
    registers and puts the token's own k and v into its key block and into the page); otherwise the
    rotation kernel runs first.  ``qkv`` may be a ``SplitSum`` where ``single_token_step_is_one_kernel``."""
    global launches
    be = backend()
    shares = None
    if isinstance(qkv, SplitSum):
        if qkv.shares.shape[0] <= 8 and single_token_step_is_one_kernel(ctx, out.dtype, heads, kv_heads, head_dim):
            shares = qkv.shares
            qkv = torch.empty(tuple(qkv.shape), dtype=out.dtype, device=out.device)     # for its shape only
        else:
            qkv = qkv.dense(out.dtype)
    if single_token_step_is_one_kernel(ctx, qkv.dtype, heads, kv_heads, head_dim):
        launches += 1
        w = int(window) if window else 0
        span = ctx.max_kv_len if not w else min(ctx.max_kv_len, w + 31)
        splits, run, scratch = _decode_plan(ctx.n_seqs * kv_heads, span, qkv.device, getattr(ctx, "min_kv_len", 0))
        part_o = part_ml = counters = None
        if scratch or splits > 8:
            part_o = torch.empty((splits, ctx.n_tokens, heads, head_dim), dtype=torch.float32, device=qkv.device)
            part_ml = torch.empty((splits, ctx.n_tokens, heads, 2), dtype=torch.float32, device=qkv.device)
            counters = _attention_counters(qkv.device, ctx.n_seqs * kv_heads)
        long_runs = _decode_long_runs(ctx.n_seqs * kv_heads, span, splits, run, head_dim, qkv.device)
        be.attention_decode(qkv, out, k_cache, v_cache, ctx.cu_q, ctx.q_start, block_table, heads, kv_heads, head_dim, w,
                            float(scale), splits, part_o, part_ml, counters, True, cos_sin, bool(store), status, shares,
                            long_runs, run)
        return out
    rope_store(qkv, ctx.positions, cos_sin, k_cache, v_cache, ctx.token_seq, block_table, heads, kv_heads, head_dim,
               store=store, status=status)
    return paged_attention(qkv, out, k_cache, v_cache, ctx, block_table, heads, kv_heads, head_dim, window, scale,
                           status=status)


FUSE_ROPE = True    # False: always the separate rotation kernel (tests compare the two)


def gate_into(src: torch.Tensor, y: torch.Tensor, gate_col: int, gate: str, dst: torch.Tensor, dst_col: int, scale: float, heads: int,
              v_dim: int) -> torch.Tensor:
    """dst[:, dst_col + h * v_dim + i] = scale * src[:, h * v_dim + i] * sigmoid(g) with g = y[:, gate_col + h] (``gate`` "head")
    or y[:, gate_col + h * v_dim + i] ("element"); "none": the scale alone.  32-bit, one rounding."""
    backend().gate_into(src, y, int(gate_col), _ATTENTION_GATES[gate], dst, int(dst_col), float(scale), int(heads), int(v_dim))
    return dst


def tensor_core_attention_takes_extras(dtype, heads: int, kv_heads: int, head_dim: int, v_dim: int, page_size: int) -> bool:
    """Whether ``paged_attention`` takes ``sinks`` and ``softcap`` at these sizes (the mma.sync kernel's)."""
    return (dtype == torch.bfloat16 and v_dim == head_dim and page_size % 16 == 0 and ATTENTION_KERNEL in ("auto", "mma")
            and backend().attention_mma_supports(head_dim, heads, kv_heads, 1)
            and backend().attention_mma_supports(head_dim, heads, kv_heads, 4))


MMA_TARGET_CTAS = 296     # CTAs that a step of single tokens aims at where the mma.sync kernel walks the keys (two for each SM)
MMA_MAX_SPLITS = 16       # the most runs that a sequence's keys are cut into for that
MMA_SINGLE_TOKEN_WARPS = int(os.environ.get("VTB200_MMA_SINGLE_TOKEN_WARPS", "4"))


def paged_attention(qkv, out, k_cache, v_cache, ctx, block_table, heads: int, kv_heads: int, head_dim: int,
                    window: Optional[int], scale: float, status=None, chunk: Optional[int] = None, sinks=None,
                    softcap=None) -> torch.Tensor:
    """Attention of the step's tokens over the paged keys and values of their sequences.
    ``ctx`` is the step's ``StepContext``.  bfloat16 runs on the tensor cores where the kernel
    takes the sizes (head_dim a multiple of 16 up to 128; tcgen05 for prompt portions at 64 and 128): single-token steps with the keys of a
    sequence split over several CTAs, other steps in tiles of 64 or 128 rows of (token, head of
    the group).  Everything else, and all of float32, runs the plain kernel.  ``chunk`` c adds the mask of chunks: key
    j is seen from position p only if j // c == p // c (the tensor-core kernels take it; the plain kernel does not)."""
    global launches
    be = backend()
    w = int(window) if window else 0
    c = int(chunk) if chunk else 0
    group = heads // kv_heads
    if sinks is not None or softcap:
        # ``sinks`` [heads] float32: one more term exp(sinks[h]) in the denominator; ``softcap`` c: a score becomes
        # c tanh(score / c).  The mma.sync kernel takes both: tiles of (token, head of the group) rows for portions, a tile a
        # sequence in steps of single tokens.
        if not tensor_core_attention_takes_extras(qkv.dtype, heads, kv_heads, head_dim, head_dim, k_cache.shape[2]):
            raise ValueError("paged_attention: sinks and capped scores run on the tensor cores in bfloat16 at head sizes that are "
                             "multiples of 16 up to 128; ops.attention_general takes the others")
        if (not softcap and ATTENTION_KERNEL == "auto" and ctx.max_q_len * group >= 128 and k_cache.shape[2] % 16 == 0
                and be.attention_tc_supports(head_dim, heads, kv_heads)):
            # portions long enough to fill tiles of 128 rows, a sink and no cap: the tcgen05 kernel (the sink is the start
            # of a row's scale and sum there too)
            tiles = _attention_tiles(ctx, 128 // group, qkv.device)
            be.attention_tc(qkv, out, k_cache, v_cache, ctx.cu_q, ctx.q_start, block_table, tiles, heads, kv_heads, head_dim, w,
                            float(scale), status, chunk=c, sinks=sinks)
            return out
        splits, part_o, part_ml = 1, None, None
        if ctx.max_q_len == 1:
            # (a tile a sequence; four warps bring a block of keys four times as fast as one, though one holds all its rows)
            warps, tiles = MMA_SINGLE_TOKEN_WARPS if be.attention_mma_supports(head_dim, heads, kv_heads, MMA_SINGLE_TOKEN_WARPS) else 1, None
            # few sequences leave most SMs without a CTA: every sequence's blocks of 64 keys are cut into equal runs, a CTA
            # each (the sink counts in the first), merged in the order of the runs
            blocks = max(1, -(-_key_span(ctx.max_kv_len, w, c) // 64))
            splits = max(1, min(MMA_MAX_SPLITS, MMA_TARGET_CTAS // max(1, ctx.n_seqs * kv_heads), blocks // 2))
            if splits > 1:
                part_o = torch.empty((splits, qkv.shape[0], heads, head_dim), dtype=torch.float32, device=qkv.device)
                part_ml = torch.empty((splits, qkv.shape[0], heads, 2), dtype=torch.float32, device=qkv.device)
        else:
            warps = 8 if ctx.max_q_len * group >= 128 and be.attention_mma_supports(head_dim, heads, kv_heads, 8) else 4
            tiles = _attention_tiles(ctx, (16 * warps) // group, qkv.device)
        be.attention_mma(qkv, out, k_cache, v_cache, ctx.cu_q, ctx.q_start, block_table, tiles, heads, kv_heads, head_dim, w,
                         float(scale), warps, splits, part_o, part_ml, status, chunk=c, sinks=sinks,
                         softcap=float(softcap) if softcap else 0.0)
        return out
    if qkv.dtype == torch.bfloat16 and ATTENTION_KERNEL in ("auto", "mma"):
        if ctx.max_q_len == 1 and be.attention_mma_supports(head_dim, heads, kv_heads, 1):
            span = _key_span(ctx.max_kv_len, w, c)
            splits, run, scratch = _decode_plan(ctx.n_seqs * kv_heads, span, qkv.device, getattr(ctx, "min_kv_len", 0))
            part_o = part_ml = counters = None
            if scratch or splits > 8:
                part_o = torch.empty((splits, ctx.n_tokens, heads, head_dim), dtype=torch.float32, device=qkv.device)
                part_ml = torch.empty((splits, ctx.n_tokens, heads, 2), dtype=torch.float32, device=qkv.device)
                counters = _attention_counters(qkv.device, ctx.n_seqs * kv_heads)
            long_runs = _decode_long_runs(ctx.n_seqs * kv_heads, span, splits, run, head_dim, qkv.device)
            be.attention_decode(qkv, out, k_cache, v_cache, ctx.cu_q, ctx.q_start, block_table, heads, kv_heads,
                                head_dim, w, float(scale), splits, part_o, part_ml, counters, long_runs=long_runs,
                                run_blocks=run, chunk=c)
            return out
        # portions long enough to fill tiles of 128 rows: the tcgen05 kernel where it takes the sizes
        if (ATTENTION_KERNEL == "auto" and ctx.max_q_len * group >= 128
                and be.attention_tc_supports(head_dim, heads, kv_heads) and k_cache.shape[2] % 16 == 0):
            # A mixed step: the single tokens at the head of the batch (a scheduler puts the decoding requests first)
            # would each be a tile of 128 rows with 7 of them live, its keys walked by one CTA.  They go to the
            # single-token kernel instead, which cuts their keys over CTAs; the two launches write disjoint rows.
            lead = _leading_single_tokens(ctx)
            if lead >= MIXED_STEP_MIN_SINGLES and be.attention_mma_supports(head_dim, heads, kv_heads, 1):
                longest = max(s.start + 1 for s in ctx.seqs[:lead])
                span = _key_span(longest, w, c)
                splits, run, scratch = _decode_plan(lead * kv_heads, span, qkv.device)
                part_o = part_ml = counters = None
                if scratch or splits > 8:
                    part_o = torch.empty((splits, lead, heads, head_dim), dtype=torch.float32, device=qkv.device)
                    part_ml = torch.empty((splits, lead, heads, 2), dtype=torch.float32, device=qkv.device)
                    counters = _attention_counters(qkv.device, lead * kv_heads)
                long_runs = _decode_long_runs(lead * kv_heads, span, splits, run, head_dim, qkv.device)
                launches += 1
                be.attention_decode(qkv[:lead], out[:lead], k_cache, v_cache, ctx.cu_q[:lead + 1], ctx.q_start[:lead],
                                    block_table[:lead], heads, kv_heads, head_dim, w, float(scale), splits, part_o, part_ml,
                                    counters, long_runs=long_runs, run_blocks=run, chunk=c)
            else:
                lead = 0
            tiles = _attention_tiles(ctx, 128 // group, qkv.device, first_seq=lead)
            be.attention_tc(qkv, out, k_cache, v_cache, ctx.cu_q, ctx.q_start, block_table, tiles, heads, kv_heads,
                            head_dim, w, float(scale), status, chunk=c)
            return out
        # mma.sync tiles of 128 rows (8 warps) where the portions are long enough to fill them, else of 64
        warps = 8 if ctx.max_q_len * group >= 128 and be.attention_mma_supports(head_dim, heads, kv_heads, 8) else 4
        if be.attention_mma_supports(head_dim, heads, kv_heads, warps):
            tiles = _attention_tiles(ctx, (16 * warps) // group, qkv.device)
            be.attention_mma(qkv, out, k_cache, v_cache, ctx.cu_q, ctx.q_start, block_table, tiles, heads, kv_heads,
                             head_dim, w, float(scale), warps, 1, None, None, status, chunk=c)
            return out
    if c:
        raise ValueError("paged_attention: the plain kernel has no mask of chunks; ops.attention_general has")
    be.attention_simt(qkv, out, k_cache, v_cache, ctx.positions, ctx.token_seq, block_table, heads, kv_heads,
                      head_dim, w, float(scale), status)
    return out


def _key_span(longest: int, window: int, chunk: int) -> int:
    """The most keys a token of a step can see, for the plan of a single-token step's CTAs."""
    span = longest if not window else min(longest, window + 31)
    return min(span, chunk) if chunk else span


_sm_counts = {}
_counters = {}


DECODE_BLOCK = 16         # keys in a block of the single-token attention kernel (one warp's unit of work)
# CTAs a step's attention aims at, in SMs (the fixed cost of a CTA against the spread of the work): where the runs of
# a sequence are a thread-block cluster, and where they meet in scratch memory
DECODE_CTAS_PER_SM = float(os.environ.get("VTB200_DECODE_CTAS_PER_SM", "0.65"))
DECODE_CTAS_PER_SM_LONG = float(os.environ.get("VTB200_DECODE_CTAS_PER_SM_LONG", "1.5"))
DECODE_MIN_RUN = int(os.environ.get("VTB200_DECODE_MIN_RUN", "8"))        # blocks below which a run of keys is not cut further
DECODE_MIN_RUN_LONG = int(os.environ.get("VTB200_DECODE_MIN_RUN_LONG", "32"))   # the same where the runs meet in scratch memory
DECODE_LONG_BOUND = int(os.environ.get("VTB200_DECODE_LONG_BOUND", "4096"))   # keys from which the runs meet in scratch memory


def _decode_plan(pairs: int, span: int, device, floor: int = 0):
    """How a single-token step's keys are cut over CTAs: (runs a sequence at most, blocks a run, whether the runs
    meet in scratch memory).  ``pairs``: sequences times KV heads; ``span``: the most keys a sequence of the step can
    hold (the bound of a captured graph).  A sequence takes about (its blocks / blocks a run) CTAs, so that
    sequences of different lengths give CTAs of like work; a step's typical sequence is taken to hold half the bound
    (a graph serves lengths between half its bound and the bound at the top, shorter ones below).

    Short bounds: the runs of a sequence are the CTAs of a thread-block cluster, which merge through shared memory;
    the cluster is sized for the typical sequence (a CTA without keys still has to be placed and to wait at the
    cluster's barriers, which costs the step more than a longer run does), and longer sequences get longer runs.
    Long bounds (the lengths of a step then differ by thousands of keys): as many runs as the longest sequence needs,
    met in scratch memory and merged by the CTA that arrives last; a CTA without keys leaves at once, a sequence of
    one run stores its result itself."""
    sms = _sm_counts.get(device)
    if sms is None:
        sms = torch.cuda.get_device_properties(device).multi_processor_count
        _sm_counts[device] = sms
    blocks = max(1, -(-span // DECODE_BLOCK))
    typical = blocks / 2
    if blocks < 2 * DECODE_MIN_RUN:
        return 1, 0, False
    # ``floor``: a lower bound of the step's lengths.  Sequences of like lengths (all at least a quarter of the bound)
    # keep the cluster at any bound, if eight runs a sequence are CTAs enough: measured inside the step on a B200 (7B
    # sizes, every sequence at 3,000 to 30,000 keys), 4 to 32 sequences 3 to 14 % faster a step than through scratch
    # memory; one or two sequences, and sequences of very different lengths, are faster through scratch memory.
    like = floor > 0 and 4 * floor >= span and pairs >= 16
    if span < DECODE_LONG_BOUND or like:
        per_pair = DECODE_CTAS_PER_SM * sms / max(pairs, 1)
        if per_pair < 1.5:
            return 1, 0, False
        run = max(DECODE_MIN_RUN, int(-(-typical // per_pair)))
        splits = min(8, int(-(-typical // run)))
        return (splits, run, False) if splits > 1 else (1, 0, False)
    # (measured on a B200, every sequence at the bound: a run below 32 blocks costs a lone sequence of 8,192 keys a
    # third more (27 against 20 us), two of them twice (37 against 19); with few sequences, one CTA an SM with all
    # eight warps beats two with six (one sequence of 32,768 keys: 24 against 33 us))
    per_pair = DECODE_CTAS_PER_SM_LONG * sms / max(pairs, 1)
    run = max(DECODE_MIN_RUN_LONG, int(-(-typical // max(per_pair, 1.0))))
    splits = min(64, -(-blocks // run))
    if pairs * 16 <= sms:
        splits = min(splits, max(1, sms // pairs))
    return (splits, run, True) if splits > 1 else (1, 0, False)


# "auto" | "always" | "never": tensor-map boxes for the keys and values of single-token steps
DECODE_BOXES = os.environ.get("VTB200_DECODE_BOXES", "auto")
LONG_RUN_BLOCKS = 16     # blocks of 16 keys a warp from which the boxes pay where the CTAs run in one round


def _decode_long_runs(pairs: int, span: int, splits: int, run: int, head_dim: int, device) -> bool:
    """Whether a single-token step's keys and values come as boxes of a tensor map (head sizes 64 and 128):
    a box arrives later than a cp.async copy but costs the warp one instruction, not 32, so it pays where a
    warp streams many blocks (16 or more: 64 sequences of 4,096 keys, a step of 5.78 against 5.94 ms); it loses
    where a warp has few, however many CTAs there are (head size 128, 24 to 128 sequences of 1,040 keys: steps 0.2
    to 1.8 % slower with boxes, measured inside the step)."""
    if head_dim not in (64, 128) or DECODE_BOXES == "never":
        return False
    if DECODE_BOXES == "always":
        return True
    sms = _sm_counts.get(device, 148)
    if head_dim == 64 and pairs * splits > sms:
        # (blocks of half the bytes: the copies' 16 instructions a lane weigh more; 256 sequences of 512 keys at
        # 0.5B sizes: a step of 1.84 ms with boxes against 1.97)
        return True
    warps = 6 if pairs * splits > sms else 8            # the kernel's shape: two CTAs an SM, or one
    blocks = max(1, -(-span // DECODE_BLOCK))
    # (the bound is that of a captured graph: a typical sequence holds half of it, as in _decode_plan)
    return (run if run else blocks // 2) >= LONG_RUN_BLOCKS * warps


def _attention_counters(device, n: int) -> torch.Tensor:
    """Arrival counters of the decode attention's runs: zero, and left zero by every launch."""
    c = _counters.get(device)
    if c is None or c.numel() < n:
        c = torch.zeros(max(n, 1 << 16), dtype=torch.int32, device=device)
        _counters[device] = c
    return c


# --------------------------------------------------------------------------- sampling


def argmax(logits: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    backend().argmax(logits, out)
    return out


def sample(logits, temperature, top_k, top_p, u, out) -> torch.Tensor:
    backend().sample(logits, temperature, top_k, top_p, u, out)
    return out


def _counted(fn):
    import functools

    @functools.wraps(fn)
    def wrapper(*a, **k):
        global launches
        launches += 1
        return fn(*a, **k)
    return wrapper


for _name in ("gate_into", "gated_delta_scan", "conv_tail_update", "memory_scan", "normed_sum", "add_rows", "embedding", "logits_scale_cap", "rmsnorm", "layernorm", "polynorm", "scale_into", "head_norm_gate", "gla_scan", "delta_scan", "retention_scan", "route_experts", "attention_differential", "route_topk", "expert_lists", "gather_picks", "combine_picks",
              "token_shift", "latent_prepare", "head_matmul", "attention_latent", "xielu", "gate_clamp", "attention_prepare", "attention_general", "silu_mul", "rope_store", "linear", "paged_attention", "argmax", "sample"):  # the others count where they launch
    globals()[_name] = _counted(globals()[_name])
