"""The arrangement of parts in a layer."""
from __future__ import annotations

import torch

from .base import Block, ParamSpec, StateSpec, build_part, register_part


@register_part("block", "prenorm")
class PreNormBlock(Block):
    """x += mixer(norm1(x)); x += ffn(norm2(x))
    (the order of v1/models/qwen2-7b/inference_fp16.dag:287-345).  The two sums are formed
    in 32-bit inside the next norm (``ResidualStream``)."""

    def __init__(self, spec, prefix, rt):
        super().__init__(spec, prefix, rt)
        self.norm1 = build_part("norm", spec.norm1, prefix + spec.norm1_name, rt)
        self.mixer = build_part("mixer", spec.mixer, prefix + spec.mixer_prefix, rt)
        self.norm2 = self.ffn = None
        if spec.ffn is not None:            # a layer without a feed-forward has the first sublayer only
            self.norm2 = build_part("norm", spec.norm2, prefix + spec.norm2_name, rt)
            self.ffn = build_part("feed_forward", spec.ffn, prefix + spec.ffn_prefix, rt)
        self.parts = tuple(p for p in (self.norm1, self.mixer, self.norm2, self.ffn) if p is not None)

    def cache_spec(self):
        return self.mixer.cache_spec()

    @property
    def graph_safe(self):
        return all(p.graph_safe for p in self.parts)

    def param_specs(self):
        out = {}
        for p in self.parts:
            out.update(p.param_specs())
        return out

    def load(self, get) -> None:
        for p in self.parts:
            p.load(get)

    def weight_bytes(self) -> int:
        return sum(p.weight_bytes() for p in self.parts)

    def first_product(self):
        return self.mixer.first_product()

    def link(self, then) -> None:
        if self.ffn is None:
            self.mixer.then = then
            return
        self.mixer.then = self.ffn.first_product()
        self.ffn.then = then

    def forward(self, stream, ctx, cache):
        h = stream.normed(self.norm1)
        stream.add(self.mixer.forward(h, ctx, cache))
        if self.ffn is None:
            return
        h = stream.normed(self.norm2)
        stream.add(self.ffn.forward(h, ctx))


@register_part("block", "sandwich")
class SandwichBlock(PreNormBlock):
    """x += m * post1(mixer(norm1(x))); x += m * post2(ffn(norm2(x))): every sublayer's result is normed (root mean
    square, weight) and multiplied by m before the residual sum.  The norm that reads the stream next does all of it
    in one pass: it norms and scales the pending result in 32-bit, adds it, and norms the sum."""

    def __init__(self, spec, prefix, rt):
        super().__init__(spec, prefix, rt)
        if spec.post1 is None or (spec.ffn is not None and spec.post2 is None):
            raise ValueError("sandwich block: a norm for each sublayer's result (post1, post2)")
        for n in (spec.post1, spec.post2):
            if n is not None and n.kind != "rmsnorm":
                raise ValueError(f"sandwich block: the norm of a sublayer's result is a root-mean-square norm, not '{n.kind}'")
        self.post1 = build_part("norm", spec.post1, prefix + spec.post1_name, rt)
        self.post2 = build_part("norm", spec.post2, prefix + spec.post2_name, rt) if spec.ffn is not None else None
        self.parts = self.parts + tuple(p for p in (self.post1, self.post2) if p is not None)

    def forward(self, stream, ctx, cache):
        s = self.spec
        h = stream.normed(self.norm1)
        stream.add(self.mixer.forward(h, ctx, cache), post=(self.post1.weighted(), s.post1.eps, s.residual_mult))
        if self.ffn is None:
            return
        h = stream.normed(self.norm2)
        stream.add(self.ffn.forward(h, ctx), post=(self.post2.weighted(), s.post2.eps, s.residual_mult))


@register_part("block", "postnorm")
class PostNormBlock(Block):
    """x <- norm1(a x + mixer(shift(x))); x <- norm2(a x + ffn(x)): the norms come after the sums and their result is the
    stream, which stays 32-bit (the norm's kernel scales the stream, adds the sublayer's result, norms the sum and puts the
    unrounded row back; the sublayer that reads it next gets a copy in the compute dtype from the same pass).  With a
    ``shift_name`` the mixer reads h_t + (h_(t-1) - h_t) * mu, h_(t-1) the stream's row of the token before, which the
    layer keeps for each request beside what its mixer keeps: the first of the run's cache slots is that row."""

    def __init__(self, spec, prefix, rt):
        super().__init__(spec, prefix, rt)
        self.norm1 = build_part("norm", spec.norm1, prefix + spec.norm1_name, rt)
        self.mixer = build_part("mixer", spec.mixer, prefix + spec.mixer_prefix, rt)
        self.norm2 = self.ffn = None
        if spec.ffn is not None:
            self.norm2 = build_part("norm", spec.norm2, prefix + spec.norm2_name, rt)
            self.ffn = build_part("feed_forward", spec.ffn, prefix + spec.ffn_prefix, rt)
        for n in (self.norm1, self.norm2):
            if n is not None and not getattr(n, "takes_stream", False):
                raise ValueError(f"postnorm block: norm '{n.spec.kind}' cannot leave its result in the stream")
        self.parts = tuple(p for p in (self.norm1, self.mixer, self.norm2, self.ffn) if p is not None)
        self.mu = None

    def cache_spec(self):
        inner = self.mixer.cache_spec()
        if self.spec.shift_name is None:
            return inner
        kept = () if inner is None else (tuple(inner) if isinstance(inner, (tuple, list)) else (inner,))
        return (StateSpec((self.spec.norm1.size,), torch.float32),) + kept

    @property
    def graph_safe(self):
        return all(p.graph_safe for p in self.parts)

    def param_specs(self):
        out = {}
        for p in self.parts:
            out.update(p.param_specs())
        if self.spec.shift_name is not None:
            out[self.prefix + self.spec.shift_name] = ParamSpec((self.spec.norm1.size,), role="vector", init="unit_uniform")
        return out

    def load(self, get) -> None:
        for p in self.parts:
            p.load(get)
        if self.spec.shift_name is not None:
            self.mu = self.rt.param(get(self.prefix + self.spec.shift_name), "vector")

    def weight_bytes(self) -> int:
        return sum(p.weight_bytes() for p in self.parts) + (0 if self.mu is None else 4 * self.mu.numel())

    def first_product(self):
        return self.mixer.first_product()

    def link(self, then) -> None:
        if self.ffn is None:
            self.mixer.then = then
            return
        self.mixer.then = self.ffn.first_product()
        self.ffn.then = then

    def forward(self, stream, ctx, cache):
        s, ops, x = self.spec, self.rt.ops, stream.x
        if stream.pending is not None:
            raise RuntimeError("postnorm block: the stream holds a delta that no norm has added")
        if s.shift_name is not None:
            views = cache if isinstance(cache, (tuple, list)) else (cache,)
            shift, rest = views[0], tuple(views[1:])
            cache = None if not rest else (rest[0] if len(rest) == 1 else rest)
            h = torch.empty(x.shape, dtype=self.rt.dtype, device=x.device)
            ops.token_shift(x, self.mu, shift.state, ctx, h, status=ctx.status)
        else:
            h = x if self.rt.dtype == torch.float32 else x.to(self.rt.dtype)
        delta = self.mixer.forward(h, ctx, cache)
        h = self.norm1.after_sum(x, delta, s.stream_scale, want_copy=self.ffn is not None, status=ctx.status)
        if self.ffn is None:
            return
        delta = self.ffn.forward(h, ctx)
        self.norm2.after_sum(x, delta, s.stream_scale, want_copy=False, status=ctx.status)
