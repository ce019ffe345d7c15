"""Mixers that carry a matrix of fixed size for each request and head instead of keys and values: gated linear
attention, the generalized delta rule, the delta rule with one decay a head and the matrix memory with exponential
gates.  The state lives in 32-bit in a ``StateSpec`` slot of the cache manager
(zero when a request is admitted), and one kernel walks a step's tokens of every (request, head) in order, a single
decoded token and a portion of a prompt alike."""
from __future__ import annotations

import torch

from .base import ParamSpec, StateSpec, build_part, register_part
from .projected import ProjectedMixer


class _Recurrent(ProjectedMixer):
    def release_unpacked(self) -> None:
        self._in = self.w_o = None

    def in_matrices(self):
        return list(self._in)

    def out_matrix(self):
        return self.w_o

    def extra_weight_bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in self._small)


@register_part("mixer", "gla")
class GatedLinearAttention(_Recurrent):
    """See ``GatedLinearAttentionSpec``.  Projections q, k, v, gate and the first low-rank matrix are one product;
    the scan kernel forms the decay (second low-rank matrix, bias, log-sigmoid / tau, exp: 32-bit) and walks the
    tokens; a second kernel norms each head's output and gates it."""

    def cache_spec(self):
        s = self.spec
        return StateSpec((s.heads, s.dim, s.v_dim), torch.float32)

    def param_specs(self):
        s, p = self.spec, self.prefix
        q, k, v, g, o, norm, a1, a2, a2b = s.names
        hd, hv = s.heads * s.dim, s.heads * s.v_dim
        return {
            p + q: ParamSpec((hd, s.hidden)), p + k: ParamSpec((hd, s.hidden)), p + v: ParamSpec((hv, s.hidden)),
            p + g: ParamSpec((hv, s.hidden)), p + o: ParamSpec((s.hidden, hv)),
            p + norm: ParamSpec((s.v_dim,), role="vector", init="one_plus_normal"),
            p + a1: ParamSpec((-16, s.hidden)), p + a2: ParamSpec((hd, -16)), p + a2b: ParamSpec((hd,), role="vector"),
        }

    def load(self, get) -> None:
        s, p, rt = self.spec, self.prefix, self.rt
        q, k, v, g, o, norm, a1, a2, a2b = s.names
        self._in = [rt.param(get(p + n)) for n in (q, k, v, g, a1)]
        self.w_o = rt.param(get(p + o))
        self.norm = rt.param(get(p + norm), "vector")
        self.a2 = rt.param(get(p + a2), "vector")             # [heads * dim, rank], read in 32-bit by the scan
        self.a2_bias = rt.param(get(p + a2b), "vector")
        self.rank = self._in[4].shape[0]
        if self.a2.shape[1] != self.rank:
            raise ValueError(f"{p}: the two low-rank matrices of the decay have ranks {self.rank} and {self.a2.shape[1]}")
        self._small = (self.norm, self.a2, self.a2_bias)
        self.pack()

    def inner_size(self) -> int:
        return self.spec.heads * self.spec.v_dim

    def core(self, y, cols, ctx, cache, out, out_col, out_scale) -> None:
        s, ops = self.spec, self.rt.ops
        o = torch.empty((y.shape[0], s.heads * s.v_dim), dtype=torch.float32, device=y.device)
        ops.gla_scan(y, cols[0], cols[1], cols[2], cols[4], self.a2, self.a2_bias, 1.0 / s.tau, s.dim ** -0.5,
                     cache.state, ctx, o, s.heads, s.dim, s.v_dim, status=ctx.status)
        ops.head_norm_gate(o, y, cols[3], self.norm, False, s.norm_eps, "silu", out, out_col, out_scale, s.heads, s.v_dim,
                           token_seq=ctx.token_seq)


@register_part("mixer", "delta_rule")
class DeltaRule(_Recurrent):
    """See ``DeltaRuleSpec``.  Projections r, k, v, gate, removal rate and the first low-rank matrix of the decay are
    one product; the scan kernel forms decay, removal rate and unit key in 32-bit and walks the tokens; a second
    kernel norms each head's output and gates it."""

    def cache_spec(self):
        s = self.spec
        return StateSpec((s.heads, s.dim, s.dim), torch.float32)

    def param_specs(self):
        s, p = self.spec, self.prefix
        r, k, v, g, o, norm, a, ab, w1, w2, w0 = s.names
        hd = s.heads * s.dim
        out = {p + n: ParamSpec((hd, s.hidden)) for n in (r, k, v, g, a)}
        out.update({
            p + o: ParamSpec((s.hidden, hd)), p + norm: ParamSpec((hd,), role="vector", init="one_plus_normal"),
            p + ab: ParamSpec((hd,), role="vector"), p + w1: ParamSpec((-16, s.hidden)), p + w2: ParamSpec((hd, -16)),
            p + w0: ParamSpec((hd,), role="vector"),
        })
        return out

    def load(self, get) -> None:
        s, p, rt = self.spec, self.prefix, self.rt
        r, k, v, g, o, norm, a, ab, w1, w2, w0 = s.names
        self._in = [rt.param(get(p + n)) for n in (r, k, v, g, a, w1)]
        self.w_o = rt.param(get(p + o))
        self.norm = rt.param(get(p + norm), "vector")
        self.a_bias = rt.param(get(p + ab), "vector")
        self.w2 = rt.param(get(p + w2), "vector")
        self.w0 = rt.param(get(p + w0), "vector")
        self.rank = self._in[5].shape[0]
        if self.w2.shape[1] != self.rank:
            raise ValueError(f"{p}: the two low-rank matrices of the decay have ranks {self.rank} and {self.w2.shape[1]}")
        self._small = (self.norm, self.a_bias, self.w2, self.w0)
        self.pack()

    def inner_size(self) -> int:
        return self.spec.heads * self.spec.dim

    def core(self, y, cols, ctx, cache, out, out_col, out_scale) -> None:
        s, ops = self.spec, self.rt.ops
        o = torch.empty((y.shape[0], s.heads * s.dim), dtype=torch.float32, device=y.device)
        ops.delta_scan(y, cols[0], cols[1], cols[2], cols[4], cols[5], self.w2, self.w0, self.a_bias, s.decay_rate,
                       s.key_eps, cache.state, ctx, o, s.heads, s.dim, status=ctx.status)
        ops.head_norm_gate(o, y, cols[3], self.norm, True, s.norm_eps, "sigmoid", out, out_col, out_scale, s.heads, s.dim,
                           token_seq=ctx.token_seq)


@register_part("mixer", "retention")
class Retention(_Recurrent):
    """See ``RetentionSpec``.  Projections q, k, v and gate are one product; the scan kernel rotates q and k in 32-bit
    while it stages them, scales k and walks the tokens with the head's decay; a second kernel norms each head's
    output (no weight) and gates it."""

    def __init__(self, spec, prefix, rt):
        super().__init__(spec, prefix, rt)
        if len(spec.decay) != spec.heads:
            raise ValueError(f"retention: {len(spec.decay)} decays for {spec.heads} heads")
        if spec.position.kind not in ("rotary_computed", "none"):
            raise ValueError(f"retention: position encoding '{spec.position.kind}' is not built; known: rotary_computed, none")
        if spec.position.kind != "none" and (spec.position.dim % 2 or spec.position.dim > spec.dim):
            raise ValueError(f"retention: the rotation covers {spec.position.dim} dimensions; it must be even and at most "
                             f"the head's {spec.dim}")
        self.position = build_part("position", spec.position, prefix, rt)

    def cache_spec(self):
        s = self.spec
        return StateSpec((s.heads, s.dim, s.v_dim), torch.float32)

    def param_specs(self):
        s, p = self.spec, self.prefix
        q, k, v, g, o = s.names
        hd, hv = s.heads * s.dim, s.heads * s.v_dim
        return {p + q: ParamSpec((hd, s.hidden)), p + k: ParamSpec((hd, s.hidden)), p + v: ParamSpec((hv, s.hidden)),
                p + g: ParamSpec((hv, s.hidden)), p + o: ParamSpec((s.hidden, hv))}

    def load(self, get) -> None:
        s, p, rt = self.spec, self.prefix, self.rt
        q, k, v, g, o = s.names
        self._in = [rt.param(get(p + n)) for n in (q, k, v, g)]
        self.w_o = rt.param(get(p + o))
        self.decay = torch.tensor(list(s.decay), dtype=torch.float64).to(torch.float32).to(rt.device)
        self.ones = torch.ones(s.v_dim, dtype=torch.float32, device=rt.device)      # the heads' norm has no weight
        self._small = (self.decay,)
        self.position.load(get)
        self.pack()

    def inner_size(self) -> int:
        return self.spec.heads * self.spec.v_dim

    def core(self, y, cols, ctx, cache, out, out_col, out_scale) -> None:
        s, ops = self.spec, self.rt.ops
        o = torch.empty((y.shape[0], s.heads * s.v_dim), dtype=torch.float32, device=y.device)
        ops.retention_scan(y, cols[0], cols[1], cols[2], self.decay, s.dim ** -0.5, getattr(self.position, "frequencies", None),
                           cache.state, ctx, o, s.heads, s.dim, s.v_dim, status=ctx.status)
        ops.head_norm_gate(o, y, cols[3], self.ones, False, s.norm_eps, "silu", out, out_col, out_scale, s.heads, s.v_dim,
                           token_seq=ctx.token_seq)


@register_part("mixer", "lightning")
class Lightning(_Recurrent):
    """See ``LightningSpec``.  Projections q, k, v and gate are one product; the scan kernel passes q, k and v through silu
    in 32-bit while it stages them and walks the tokens with the head's decay (the retention walk without a rotation or a
    scale of k); a second kernel norms the heads' results together, multiplies by the weight and by sigmoid(gate)."""

    def __init__(self, spec, prefix, rt):
        super().__init__(spec, prefix, rt)
        if len(spec.decay) != spec.heads:
            raise ValueError(f"lightning: {len(spec.decay)} decays for {spec.heads} heads")

    def cache_spec(self):
        s = self.spec
        return StateSpec((s.heads, s.dim, s.v_dim), torch.float32)

    def param_specs(self):
        s, p = self.spec, self.prefix
        q, k, v, g, o, norm = s.names
        hd, hv = s.heads * s.dim, s.heads * s.v_dim
        return {p + q: ParamSpec((hd, s.hidden)), p + k: ParamSpec((hd, s.hidden)), p + v: ParamSpec((hv, s.hidden)),
                p + g: ParamSpec((hv, s.hidden)), p + o: ParamSpec((s.hidden, hv)),
                p + norm: ParamSpec((hv,), role="vector", init="one_plus_normal")}

    def load(self, get) -> None:
        s, p, rt = self.spec, self.prefix, self.rt
        q, k, v, g, o, norm = s.names
        self._in = [rt.param(get(p + n)) for n in (q, k, v, g)]
        self.w_o = rt.param(get(p + o))
        self.norm = rt.param(get(p + norm), "vector")
        self.decay = torch.tensor(list(s.decay), dtype=torch.float64).to(torch.float32).to(rt.device)
        self._small = (self.decay, self.norm)
        self.pack()

    def inner_size(self) -> int:
        return self.spec.heads * self.spec.v_dim

    def core(self, y, cols, ctx, cache, out, out_col, out_scale) -> None:
        s, ops = self.spec, self.rt.ops
        n = s.heads * s.v_dim
        o = torch.empty((y.shape[0], n), dtype=torch.float32, device=y.device)
        ops.retention_scan(y, cols[0], cols[1], cols[2], self.decay, 1.0, None, cache.state, ctx, o, s.heads, s.dim, s.v_dim,
                           status=ctx.status, act=True)
        # the heads are normed together: one "head" as wide as all of them, with a weight for every channel
        ops.head_norm_gate(o, y, cols[3], self.norm, True, s.norm_eps, "sigmoid", out, out_col, out_scale, 1, n,
                           token_seq=ctx.token_seq)


def _conv_taps(shape, g, sigma, device):
    """The taps of a short convolution in the random-weights mode: of the order of a half whatever sigma is, so that every
    tap counts."""
    return torch.randn(shape, generator=g, dtype=torch.float32, device=device) * 0.4


def _register_conv_taps():
    from ..weights.loader import register_initialiser
    register_initialiser("conv_taps", _conv_taps, replace=True)


_register_conv_taps()


@register_part("mixer", "gated_delta")
class GatedDelta(_Recurrent):
    """See ``GatedDeltaSpec``.  Projections q, k, v, gate and the two matrices of beta and of the decay are one product; the
    scan kernel passes q, k and v through their convolutions and silu while it stages them (their inputs before the step's
    first token come from the request's kept inputs), forms unit q and k, beta and the decay in 32-bit and walks the
    tokens; one kernel renews the kept inputs; one norms each head's result and gates it.  A request keeps the state
    [heads, dim, v_dim] and, with more than one tap, the last taps - 1 inputs [taps - 1, channels of q, k and v]."""

    def __init__(self, spec, prefix, rt):
        super().__init__(spec, prefix, rt)
        if spec.heads % spec.kv_heads:
            raise ValueError(f"gated delta rule: {spec.heads} heads over {spec.kv_heads} heads of q and k")
        if spec.taps < 1:
            raise ValueError("gated delta rule: a convolution has at least one tap")
        self.widths = (spec.kv_heads * spec.dim, spec.kv_heads * spec.dim, spec.heads * spec.v_dim)

    def cache_spec(self):
        s = self.spec
        state = StateSpec((s.heads, s.dim, s.v_dim), torch.float32)
        if s.taps == 1:
            return state
        return (state, StateSpec((s.taps - 1, sum(self.widths)), torch.float32))

    def param_specs(self):
        s, p, x = self.spec, self.prefix, self.spec.conv_suffix
        q, k, v, g, o, norm, b, a, a_log, dt = s.names
        nq, nk, nv = self.widths
        out = {p + q: ParamSpec((nq, s.hidden)), p + k: ParamSpec((nk, s.hidden)), p + v: ParamSpec((nv, s.hidden)),
               p + g: ParamSpec((nv, s.hidden)), p + o: ParamSpec((s.hidden, nv)),
               p + norm: ParamSpec((s.v_dim,), role="vector", init="one_plus_normal"),
               p + b: ParamSpec((s.heads, s.hidden)), p + a: ParamSpec((s.heads, s.hidden)),
               p + a_log: ParamSpec((s.heads,), role="vector"), p + dt: ParamSpec((s.heads,), role="vector")}
        out.update({p + n + x: ParamSpec((w, s.taps), role="vector", init="conv_taps") for n, w in zip((q, k, v), self.widths)})
        return out

    def load(self, get) -> None:
        s, p, rt, x = self.spec, self.prefix, self.rt, self.spec.conv_suffix
        q, k, v, g, o, norm, b, a, a_log, dt = s.names
        self._in = [rt.param(get(p + n)) for n in (q, k, v, g, b, a)]
        self.w_o = rt.param(get(p + o))
        self.norm = rt.param(get(p + norm), "vector")
        self.a_log = rt.param(get(p + a_log), "vector")
        self.dt_bias = rt.param(get(p + dt), "vector")
        self.conv = [rt.param(get(p + n + x), "vector") for n in (q, k, v)]
        self._small = (self.norm, self.a_log, self.dt_bias, *self.conv)
        self.pack()

    def inner_size(self) -> int:
        return self.spec.heads * self.spec.v_dim

    def core(self, y, cols, ctx, cache, out, out_col, out_scale) -> None:
        s, ops = self.spec, self.rt.ops
        state, tail = (cache[0].state, cache[1].state) if isinstance(cache, (tuple, list)) else (cache.state, None)
        o = torch.empty((y.shape[0], s.heads * s.v_dim), dtype=torch.float32, device=y.device)
        ops.gated_delta_scan(y, cols[0], cols[1], cols[2], cols[4], cols[5], *self.conv, self.a_log, self.dt_bias, s.key_eps,
                             s.dim ** -0.5, state, tail, ctx, o, s.heads, s.kv_heads, s.dim, s.v_dim, status=ctx.status)
        if tail is not None:
            ops.conv_tail_update(y, cols[:3], self.widths, tail, ctx, status=ctx.status)
        ops.head_norm_gate(o, y, cols[3], self.norm, False, s.norm_eps, "silu", out, out_col, out_scale, s.heads, s.v_dim,
                           token_seq=ctx.token_seq)


@register_part("mixer", "matrix_memory")
class MatrixMemory(_Recurrent):
    """See ``MatrixMemorySpec``.  Projections q, k, v, gate and the two gates' matrices are one product; the scan kernel
    forms the capped logarithms of the gates, the running maximum and the two exponentials in 32-bit and walks the tokens,
    the normalizer n as one more column of the state; a second kernel norms each head's result, multiplies by the weight
    and by sigmoid(gate).  A request keeps [heads, dim + 1, v_dim + 1]: S beside n, and m in the last row."""

    def cache_spec(self):
        s = self.spec
        return StateSpec((s.heads, s.dim + 1, s.v_dim + 1), torch.float32)

    def param_specs(self):
        s, p, bx = self.spec, self.prefix, self.spec.bias_suffix
        q, k, v, g, o, norm, i, f = s.names
        hd, hv = s.heads * s.dim, s.heads * s.v_dim
        return {p + q: ParamSpec((hd, s.hidden)), p + k: ParamSpec((hd, s.hidden)), p + v: ParamSpec((hv, s.hidden)),
                p + g: ParamSpec((hv, s.hidden)), p + o: ParamSpec((s.hidden, hv)),
                p + norm: ParamSpec((hv,), role="vector", init="one_plus_normal"),
                p + i: ParamSpec((s.heads, s.hidden)), p + f: ParamSpec((s.heads, s.hidden)),
                p + i + bx: ParamSpec((s.heads,), role="vector"), p + f + bx: ParamSpec((s.heads,), role="vector")}

    def load(self, get) -> None:
        s, p, rt, bx = self.spec, self.prefix, self.rt, self.spec.bias_suffix
        q, k, v, g, o, norm, i, f = s.names
        self._in = [rt.param(get(p + n)) for n in (q, k, v, g, i, f)]
        self.w_o = rt.param(get(p + o))
        self.norm = rt.param(get(p + norm), "vector")
        self.i_bias = rt.param(get(p + i + bx), "vector")
        self.f_bias = rt.param(get(p + f + bx), "vector")
        self._small = (self.norm, self.i_bias, self.f_bias)
        self.pack()

    def inner_size(self) -> int:
        return self.spec.heads * self.spec.v_dim

    def core(self, y, cols, ctx, cache, out, out_col, out_scale) -> None:
        s, ops = self.spec, self.rt.ops
        o = torch.empty((y.shape[0], s.heads * s.v_dim), dtype=torch.float32, device=y.device)
        ops.memory_scan(y, cols[0], cols[1], cols[2], cols[4], cols[5], self.i_bias, self.f_bias, s.gate_cap, s.dim ** -0.5,
                        s.den_eps, cache.state, ctx, o, s.heads, s.dim, s.v_dim, status=ctx.status)
        ops.head_norm_gate(o, y, cols[3], self.norm, True, s.norm_eps, "sigmoid", out, out_col, out_scale, s.heads, s.v_dim,
                           token_seq=ctx.token_seq)
