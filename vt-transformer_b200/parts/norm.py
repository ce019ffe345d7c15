"""Norms over the residual stream, with the residual sum folded in."""
from __future__ import annotations

import torch

from .base import Norm, ParamSpec, register_part


@register_part("norm", "rmsnorm")
class RMSNorm(Norm):
    """out = w * v * rsqrt(mean(v^2) + eps) with v = x (+ delta), everything in 32-bit and
    one rounding at the end; the weight multiplies as it is, not as 1 + w
    (v1/tensortype/cuda_kernels/rmsnorm.cu:20-47).  ``prefix`` is the tensor's name
    without the spec's ``weight_suffix`` (".weight")."""

    graph_safe = True
    takes_shares = True        # the kernel adds a product's unadded shares while it reads them
    takes_post = True          # ... and norms and scales the delta first where a layer asks for that
    takes_stream = True        # ... and can leave the normed row in the stream (a layer whose norm comes after the sum)

    def param_specs(self):
        init = "normal" if self.spec.one_plus else "one_plus_normal"
        return {self.prefix + self.spec.weight_suffix: ParamSpec((self.spec.size,), role="vector", init=init)}

    def load(self, get) -> None:
        self.weight = self.rt.param(get(self.prefix + self.spec.weight_suffix), "vector")
        if self.spec.one_plus:          # stored around zero: the kernels multiply with 1 + w, formed once in 32-bit
            self.weight = (self.weight + 1.0).contiguous()

    def weighted(self):
        return self.weight

    def weight_bytes(self) -> int:
        return self.weight.numel() * self.weight.element_size()

    def __call__(self, x, delta=None, rows=None, status=None, post=None):
        n = x.shape[0] if rows is None else rows.numel()
        out = torch.empty((n, self.spec.size), dtype=self.rt.dtype, device=x.device)
        return self.rt.ops.rmsnorm(x, self.weight, self.spec.eps, out, delta=delta, rows=rows, status=status, post=post,
                                   groups=self.spec.groups)

    def after_sum(self, x, delta, x_scale: float, want_copy: bool = True, status=None):
        """x <- N(x_scale * x + delta), the normed row unrounded in the 32-bit stream; returns its copy in the compute
        dtype, or None where ``want_copy`` is False and the kernel can do without the copy (a delta that is a tensor)."""
        out = None
        if want_copy or not isinstance(delta, torch.Tensor):
            out = torch.empty(x.shape, dtype=self.rt.dtype, device=x.device)
        self.rt.ops.rmsnorm(x, self.weight, self.spec.eps, out, delta=delta, status=status, groups=self.spec.groups,
                            x_scale=x_scale, to_stream=True)
        return out


@register_part("norm", "layernorm")
class LayerNorm(RMSNorm):
    """out = w * (v - mean(v)) * rsqrt(var(v) + eps) with v = x (+ delta), var the mean of the squared deviations, no
    bias; everything in 32-bit and one rounding at the end.  The kernel is the RMS norm's with the mean taken off."""

    takes_stream = False

    def __init__(self, spec, prefix, rt):
        super().__init__(spec, prefix, rt)
        if spec.groups != 1:
            raise ValueError("layernorm: groups are built for the root-mean-square norm only")

    def __call__(self, x, delta=None, rows=None, status=None, post=None):
        n = x.shape[0] if rows is None else rows.numel()
        out = torch.empty((n, self.spec.size), dtype=self.rt.dtype, device=x.device)
        return self.rt.ops.layernorm(x, self.weight, self.spec.eps, out, delta=delta, rows=rows, status=status, post=post)
