"""Feed-forwards: gated, with the PolyNorm activation, and a mixture of gated experts."""
from __future__ import annotations

import torch

from .base import FeedForward, ParamSpec, register_part


@register_part("feed_forward", "gated_mlp")
class GatedMLP(FeedForward):
    """down(silu(gate(h)) * up(h)) without biases, silu(z) = z / (1 + exp(-z)) in 32-bit
    (v1/models/qwen2-7b/inference_fp16.dag:333-337,
    v1/tensortype/cuda_kernels/silu_product.cu:15-17).  Gate and up are one product over
    the rows of the two matrices interleaved in runs of 8 (``ops.interleave_gate_up``), so
    that the activation can be formed in the product's epilogue."""

    graph_safe = True

    def __init__(self, spec, prefix, rt):
        super().__init__(spec, prefix, rt)
        if spec.activation != "silu":
            raise ValueError(f"gated_mlp: activation '{spec.activation}' is not built; known: silu")

    def param_specs(self):
        s, p, x = self.spec, self.prefix, self.spec.weight_suffix
        g, u, d = s.names
        return {
            f"{p}{g}{x}": ParamSpec((s.inter, s.hidden)),
            f"{p}{u}{x}": ParamSpec((s.inter, s.hidden)),
            f"{p}{d}{x}": ParamSpec((s.hidden, s.inter)),
        }

    def load(self, get) -> None:
        s, p, rt, x = self.spec, self.prefix, self.rt, self.spec.weight_suffix
        g, u, d = s.names
        mats = [rt.param(get(f"{p}{n}{x}")) for n in (g, u)]
        if mats[0].dtype != mats[1].dtype:
            mats = [m.float() for m in mats]
        self.w_down = rt.param(get(f"{p}{d}{x}"))
        if s.inter % 8:
            # an inner size that is no multiple of 8 is padded to one: rows of zeros in gate and up give silu(0) * 0 = 0,
            # which meets columns of zeros in down
            from .projected import pack_columns, pack_rows
            mats = [pack_rows([m])[0] for m in mats]
            self.w_down = pack_columns([self.w_down])[0]
        self.inter = mats[0].shape[0]
        self.w_gate_up = rt.ops.interleave_gate_up(mats[0], mats[1])
        del mats

    def weight_bytes(self) -> int:
        return (self.w_gate_up.numel() * self.w_gate_up.element_size()
                + self.w_down.numel() * self.w_down.element_size())

    def first_product(self):
        return self.rt.ops.product_hint(self.w_gate_up, "silu_mul")

    def forward(self, h, ctx):
        s, ops = self.spec, self.rt.ops
        T = h.shape[0]
        act = torch.empty((T, self.inter), dtype=h.dtype, device=h.device)
        ops.linear_silu_mul(h, self.w_gate_up, act, then=ops.product_hint(self.w_down, "stream"))
        return ops.linear_to_stream(act, self.w_down, None, then=self.then)


@register_part("feed_forward", "polynorm_mlp")
class PolyNormMLP(FeedForward):
    """down(act(up(h))) without biases, act(z) = a N(z) + b N(z^2) + c N(z^3) + e with N a token's inner vector
    divided by its root mean square: one kernel reads a row of up's result, forms the three mean squares in 32-bit
    and writes the activation."""

    graph_safe = True

    def param_specs(self):
        s, p = self.spec, self.prefix
        u, d, act = s.names
        return {f"{p}{u}": ParamSpec((s.inter, s.hidden)), f"{p}{d}": ParamSpec((s.hidden, s.inter)),
                f"{p}{act}": ParamSpec((4,), role="vector", init="polynorm_coefficients")}

    def load(self, get) -> None:
        s, p, rt = self.spec, self.prefix, self.rt
        u, d, act = s.names
        # an inner size that is no multiple of 8 is padded to one (rows of zeros in up, columns of zeros in down): the
        # products read rows in 16-byte pieces; the activation's means are over the real columns
        from .projected import pack_columns, pack_rows
        self.w_up, _ = pack_rows([rt.param(get(f"{p}{u}"))])
        self.w_down, _, _ = pack_columns([rt.param(get(f"{p}{d}"))])
        self.coefficients = rt.param(get(f"{p}{act}"), "vector")

    def weight_bytes(self) -> int:
        return sum(m.numel() * m.element_size() for m in (self.w_up, self.w_down, self.coefficients))

    def first_product(self):
        return self.rt.ops.product_hint(self.w_up, "linear")

    def forward(self, h, ctx):
        s, ops = self.spec, self.rt.ops
        z = torch.empty((h.shape[0], self.w_up.shape[0]), dtype=h.dtype, device=h.device)
        ops.linear(h, self.w_up, None, z, then=ops.product_hint(self.w_down, "stream"))
        ops.polynorm(z, self.coefficients, s.eps, z, n_mean=s.inter)
        return ops.linear_to_stream(z, self.w_down, None, then=self.then)


@register_part("feed_forward", "xielu_mlp")
class XieluMLP(FeedForward):
    """See ``XieluMLPSpec``: down(act(up(h) + b_up)) + b_down.  The two numbers of the activation become
    a_pos = softplus(p) and a_neg = 1/2 + softplus(q) once, when the weights are loaded; the activation's kernel works in
    32-bit on the product's result.  An inner size that is no multiple of 8 is zero-padded (act(0) = 0)."""

    graph_safe = True

    def param_specs(self):
        s, p = self.spec, self.prefix
        u, d, act = s.names
        return {f"{p}{u}": ParamSpec((s.inter, s.hidden)), f"{p}{u}{s.bias_suffix}": ParamSpec((s.inter,), role="vector"),
                f"{p}{d}": ParamSpec((s.hidden, s.inter)), f"{p}{d}{s.bias_suffix}": ParamSpec((s.hidden,), role="vector"),
                f"{p}{act}": ParamSpec((2,), role="vector")}

    def load(self, get) -> None:
        import math
        from .projected import pack_columns, pack_rows
        s, p, rt = self.spec, self.prefix, self.rt
        u, d, act = s.names
        self.w_up, _ = pack_rows([rt.param(get(f"{p}{u}"))])
        self.w_down, _, _ = pack_columns([rt.param(get(f"{p}{d}"))])
        b_up = rt.param(get(f"{p}{u}{s.bias_suffix}"), "vector")
        pad = self.w_up.shape[0] - b_up.numel()
        self.b_up = torch.cat([b_up, torch.zeros(pad, dtype=b_up.dtype, device=b_up.device)]).contiguous() if pad else b_up
        self.b_down = rt.param(get(f"{p}{d}{s.bias_suffix}"), "vector")
        two = [float(v) for v in get(f"{p}{act}").double().flatten().tolist()]
        softplus = lambda v: max(v, 0.0) + math.log1p(math.exp(-abs(v)))
        self.a_pos, self.a_neg = softplus(two[0]), 0.5 + softplus(two[1])

    def weight_bytes(self) -> int:
        return sum(m.numel() * m.element_size() for m in (self.w_up, self.w_down, self.b_up, self.b_down))

    def first_product(self):
        return self.rt.ops.product_hint(self.w_up, "linear")

    def forward(self, h, ctx):
        ops = self.rt.ops
        z = torch.empty((h.shape[0], self.w_up.shape[0]), dtype=h.dtype, device=h.device)
        ops.linear(h, self.w_up, self.b_up, z, then=ops.product_hint(self.w_down, "stream"))
        ops.xielu(z, z, self.a_pos, self.a_neg)
        return ops.linear_to_stream(z, self.w_down, self.b_down, then=self.then)


@register_part("feed_forward", "experts")
class Experts(FeedForward):
    """See ``ExpertsSpec``.  The router's logits are 32-bit dot products formed inside the routing kernel (its matrix is
    kept in 32-bit).  All experts'
    gate and up matrices, and the shared expert's, are one packed matrix, so silu(gate) * up of every expert for every
    token is ONE product with the activation in its epilogue; one kernel then picks each token's experts, forms their
    weights and multiplies the chosen experts' columns by them (zero for the others); the down matrices are packed
    along the inner dimension, so the weighted sum over the experts and the shared expert is ONE product.  A step of a
    few tokens reads every expert's weights anyway; a long portion pays experts / top times the products' work for
    two launches instead of two for every expert and no regrouping of the tokens.  So a step with many picks (tokens times
    top, ``ops.EXPERTS_GROUPED_MIN_PICKS``) that is no step of single tokens groups its tokens by expert instead: the
    picks of every token, the list of every expert's picks in rising order, the input rows sorted by expert, the two
    products of every expert over its slice of rows (the host reads the experts' counts for that: one wait a layer),
    the shared expert's two products over all rows, and one kernel that adds a token's picks with their weights in the
    order of the picks, in 32-bit.  Inner sizes that are no multiple of 8 are zero-padded.  The down matrices are kept
    twice (packed along the inner dimension for the one product, one by one for the grouped products)."""

    graph_safe = True

    def __init__(self, spec, prefix, rt):
        super().__init__(spec, prefix, rt)
        if spec.activation not in ("silu", "clamped"):
            raise ValueError(f"experts: activation '{spec.activation}' is not built; known: silu, clamped")
        if spec.router_weights not in ("softmax", "sigmoid_share"):
            raise ValueError(f"experts: router weights '{spec.router_weights}' are not built; known: softmax, sigmoid_share")

    def gate_up(self, x, w_gate_up, act, limit: float, then=None, split: int = 0, limit2=None):
        """act = what the last product multiplies, from x and the interleaved gate and up matrices: silu(gate) * up in the
        product's epilogue, or, for the clamped form, the product and then the activation's kernel."""
        s, ops = self.spec, self.rt.ops
        if s.activation == "silu":
            return ops.linear_silu_mul(x, w_gate_up, act, then=then)
        gu = torch.empty((x.shape[0], w_gate_up.shape[0]), dtype=x.dtype, device=x.device)
        ops.linear(x, w_gate_up, None, gu)
        return ops.gate_clamp(gu, act, 8, s.gate_alpha, limit, split=split, limit2=limit2)

    def param_specs(self):
        s, p = self.spec, self.prefix
        g, u, d = s.names
        out = {p + s.router_name: ParamSpec((s.experts, s.hidden))}
        blocks = [(f"{p}{s.expert_prefix}{e}.", s.inter) for e in range(s.experts)]
        if s.shared_inter:
            blocks.append((p + s.shared_prefix, s.shared_inter))
        for prefix, inter in blocks:
            out[prefix + g] = ParamSpec((inter, s.hidden))
            out[prefix + u] = ParamSpec((inter, s.hidden))
            out[prefix + d] = ParamSpec((s.hidden, inter))
        return out

    def load(self, get) -> None:
        s, p, rt = self.spec, self.prefix, self.rt
        g, u, d = s.names
        self.router = rt.param(get(p + s.router_name), "vector")       # [experts, hidden] in 32-bit
        self.inter = -(-s.inter // 8) * 8
        blocks = [(f"{p}{s.expert_prefix}{e}.", s.inter, self.inter) for e in range(s.experts)]
        if s.shared_inter:
            blocks.append((p + s.shared_prefix, s.shared_inter, -(-s.shared_inter // 8) * 8))
        gate_up, down = [], []
        for prefix, inter, padded in blocks:
            mats = [rt.param(get(prefix + n)) for n in (g, u, d)]
            if len({m.dtype for m in mats}) > 1:
                mats = [m.float() for m in mats]
            wg, wu, wd = mats
            if padded != inter:
                zeros = torch.zeros((padded - inter, s.hidden), dtype=wg.dtype, device=wg.device)
                wg, wu = torch.cat([wg, zeros]), torch.cat([wu, zeros])
                wd = torch.cat([wd, torch.zeros((s.hidden, padded - inter), dtype=wd.dtype, device=wd.device)], dim=1)
            gate_up.append(rt.ops.interleave_gate_up(wg, wu))
            down.append(wd)
        if len({m.dtype for m in gate_up + down}) > 1:
            gate_up, down = [m.float() for m in gate_up], [m.float() for m in down]
        self.w_gate_up = torch.cat(gate_up, dim=0).contiguous()
        self.w_down = torch.cat(down, dim=1).contiguous()
        # for the grouped products: every expert's matrices as contiguous [n, k] (views of the packed rows; the down
        # matrices as they were)
        rows = [g.shape[0] for g in gate_up]
        starts = [sum(rows[:i]) for i in range(len(rows))]
        self.gate_up_of = [self.w_gate_up[a:a + n] for a, n in zip(starts, rows)]
        self.down_of = [d.contiguous() for d in down]

    def weight_bytes(self) -> int:
        return sum(m.numel() * m.element_size() for m in (self.router, self.w_gate_up, self.w_down))

    def first_product(self):
        return self.rt.ops.product_hint(self.w_gate_up, "silu_mul")

    def forward(self, h, ctx):
        s, ops = self.spec, self.rt.ops
        T = h.shape[0]
        if ctx.max_q_len > 1 and T * s.top >= ops.EXPERTS_GROUPED_MIN_PICKS:
            return self.grouped(h)
        act = torch.empty((T, self.w_down.shape[1]), dtype=h.dtype, device=h.device)
        self.gate_up(h, self.w_gate_up, act, s.limit, then=ops.product_hint(self.w_down, "stream"),
                     split=s.experts * self.inter, limit2=s.shared_limit if s.shared_inter else None)
        # the router's logits are formed there, in 32-bit
        ops.route_experts(None, s.top, act, self.inter, x=h, router=self.router, weights_by=s.router_weights, scale=s.router_scale)
        return ops.linear_to_stream(act, self.w_down, None, then=self.then)

    def grouped(self, h):
        """The tokens grouped by expert (see the class)."""
        s, ops, dev = self.spec, self.rt.ops, h.device
        T, picks = h.shape[0], h.shape[0] * s.top
        ids = torch.empty((T, s.top), dtype=torch.int32, device=dev)
        weights = torch.empty((T, s.top), dtype=torch.float32, device=dev)
        ops.route_topk(None, s.top, ids, weights, x=h, router=self.router, weights_by=s.router_weights, scale=s.router_scale)
        lists = torch.empty((s.experts, T), dtype=torch.int32, device=dev)
        counts = torch.empty((s.experts,), dtype=torch.int32, device=dev)
        ops.expert_lists(ids, lists, counts)
        rows = torch.empty((picks, s.hidden), dtype=h.dtype, device=dev)
        where = torch.empty((picks,), dtype=torch.int32, device=dev)
        ops.gather_picks(h, lists, counts, s.top, rows, where)
        shared_y = None
        if s.shared_inter:          # the shared expert's products are enqueued before the host waits for the counts
            act = torch.empty((T, self.down_of[-1].shape[1]), dtype=h.dtype, device=dev)
            self.gate_up(h, self.gate_up_of[-1], act, s.shared_limit)
            shared_y = torch.empty((T, s.hidden), dtype=h.dtype, device=dev)
            ops.linear(act, self.down_of[-1], None, shared_y)
        act = torch.empty((picks, self.inter), dtype=h.dtype, device=dev)
        y = torch.empty((picks, s.hidden), dtype=h.dtype, device=dev)
        at = 0
        for e, n in enumerate(counts.tolist()):
            if n:
                self.gate_up(rows[at:at + n], self.gate_up_of[e], act[at:at + n], s.limit)
                ops.linear(act[at:at + n], self.down_of[e], None, y[at:at + n])
            at += n
        out = torch.empty((T, s.hidden), dtype=h.dtype, device=dev)
        return ops.combine_picks(y, where, weights, shared_y, out)
