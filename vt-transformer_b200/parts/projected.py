"""Mixers of the shape  projections of h -> a core on the projected values -> one output projection,  and the
mixer that runs several of them side by side.

Such a mixer says which matrices it multiplies its input with (``in_matrices``), how wide what its core leaves for
the output projection is (``inner_size``), and with which matrix that is projected (``out_matrix``).  Alone it runs
one product over its packed input matrices, its core, and the output product.  Side by side (``ParallelMixer``) the
branches share both products: one over all branches' input matrices, and one over their output matrices packed along
the inner dimension, so that sum_i scale_i * O_i core_i costs one product whose inputs the cores have scaled.
"""
from __future__ import annotations

from typing import List, Optional

import torch

from .base import Mixer, build_part, register_part

PACK = 8    # column ranges of packed products start at multiples of 8 (16 bytes of bfloat16)


def _round_up(n: int, to: int = PACK) -> int:
    return -(-n // to) * to


def pack_rows(mats: List[torch.Tensor]):
    """The matrices [n_i, k] one below the other, each padded with zero rows to a multiple of 8.  Returns the packed
    matrix and the first row of each."""
    if len({m.dtype for m in mats}) > 1:
        mats = [m.float() for m in mats]
    parts, starts, at = [], [], 0
    for m in mats:
        starts.append(at)
        parts.append(m)
        pad = _round_up(m.shape[0]) - m.shape[0]
        if pad:
            parts.append(torch.zeros((pad, m.shape[1]), dtype=m.dtype, device=m.device))
        at += m.shape[0] + pad
    return torch.cat(parts, dim=0).contiguous(), starts


def pack_columns(mats: List[torch.Tensor]):
    """The matrices [n, k_i] side by side, each padded with zero columns to a multiple of 8."""
    if len({m.dtype for m in mats}) > 1:
        mats = [m.float() for m in mats]
    parts, starts, at = [], [], 0
    for m in mats:
        starts.append(at)
        parts.append(m)
        pad = _round_up(m.shape[1]) - m.shape[1]
        if pad:
            parts.append(torch.zeros((m.shape[0], pad), dtype=m.dtype, device=m.device))
        at += m.shape[1] + pad
    return torch.cat(parts, dim=1).contiguous(), starts, at


def pack_biases(mats: List[torch.Tensor], biases) -> Optional[torch.Tensor]:
    """The biases of the matrices that ``pack_rows`` packs, as one float32 vector with zeros where a matrix has none and
    in the padding; None if no matrix has a bias."""
    if biases is None or all(b is None for b in biases):
        return None
    parts = []
    for m, b in zip(mats, biases):
        n = _round_up(m.shape[0])
        v = torch.zeros(n, dtype=torch.float32, device=m.device)
        if b is not None:
            v[:m.shape[0]] = b.float()
        parts.append(v)
    return torch.cat(parts).contiguous()


def count_kept(spec) -> int:
    """How many cache views a mixer with this ``cache_spec()`` takes."""
    if spec is None:
        return 0
    return len(spec) if isinstance(spec, (tuple, list)) else 1


def take_views(views: list, spec):
    """The next views of ``views`` for a mixer with this ``cache_spec()``: None, one view, or a tuple of them."""
    n = count_kept(spec)
    if n == 0:
        return None
    mine = [views.pop(0) for _ in range(n)]
    return tuple(mine) if isinstance(spec, (tuple, list)) else mine[0]


class ProjectedMixer(Mixer):
    """``in_matrices()``: after ``load``, the matrices [n_i, hidden] of the projections the core reads, in the order
    in which ``core`` finds their results: result i starts at column ``cols[i]`` of ``y``.
    ``core(y, cols, ctx, cache, out, out_col, out_scale)``: y [T, N] holds the projections; the core writes
    out_scale * (what the output projection multiplies) into out[:, out_col : out_col + inner_size()].
    ``out_matrix()``: [hidden, inner_size()].  ``in_biases()``: None, or for every matrix of ``in_matrices()`` its bias
    (float32) or None; ``out_bias()``: the output projection's bias or None."""

    graph_safe = True
    standalone = True       # False for a branch of a ``ParallelMixer``, which packs its branches' matrices itself

    def in_matrices(self) -> List[torch.Tensor]:
        raise NotImplementedError

    def inner_size(self) -> int:
        raise NotImplementedError

    def out_matrix(self) -> torch.Tensor:
        raise NotImplementedError

    def core(self, y, cols, ctx, cache, out, out_col: int, out_scale: float) -> None:
        raise NotImplementedError

    def in_biases(self):
        return None

    def out_bias(self):
        return None

    # ---- alone ---------------------------------------------------------------------------
    def pack(self) -> None:
        """Packs the matrices for a run of this mixer alone (a ``ParallelMixer`` packs its branches' itself)."""
        if not self.standalone:
            return
        self.w_in, self.cols = pack_rows(self.in_matrices())
        self.b_in = pack_biases(self.in_matrices(), self.in_biases())
        self.w_out, _, self.k_out = pack_columns([self.out_matrix()])
        self.b_out = self.out_bias()
        self.release_unpacked()

    def release_unpacked(self) -> None:
        """Drops the single matrices once a packed copy exists."""

    def weight_bytes(self) -> int:
        return (sum(m.numel() * m.element_size() for m in (self.w_in, self.w_out, self.b_in, self.b_out) if m is not None)
                + self.extra_weight_bytes())

    def extra_weight_bytes(self) -> int:
        return 0

    def first_product(self):
        return self.rt.ops.product_hint(self.w_in, "linear")

    def forward(self, h, ctx, cache):
        ops = self.rt.ops
        T = h.shape[0]
        y = torch.empty((T, self.w_in.shape[0]), dtype=h.dtype, device=h.device)
        ops.linear(h, self.w_in, self.b_in, y)
        padded = self.k_out != self.inner_size()
        act = (torch.zeros if padded else torch.empty)((T, self.k_out), dtype=h.dtype, device=h.device)
        self.core(y, self.cols, ctx, cache, act, 0, 1.0)
        return ops.linear_to_stream(act, self.w_out, self.b_out, then=self.then)


@register_part("mixer", "parallel")
class ParallelMixer(Mixer):
    """sum_i scales[i] * branches[i](h): every branch a ``ProjectedMixer``.  One product over all branches' input
    matrices, the cores one after the other (each scaling what it leaves by its branch's scale, in 32-bit, before
    the one rounding), one product over the output matrices packed along the inner dimension.  What the branches
    keep between steps is handed on as a tuple, one entry for each branch that keeps something."""

    def __init__(self, spec, prefix, rt):
        super().__init__(spec, prefix, rt)
        if not (len(spec.branches) == len(spec.scales) == len(spec.prefixes)) or not spec.branches:
            raise ValueError("parallel mixer: one scale and one prefix for each branch")
        self.branches = [build_part("mixer", b, prefix + p, rt) for b, p in zip(spec.branches, spec.prefixes)]
        for b in self.branches:
            b.standalone = False
            if not isinstance(b, ProjectedMixer):
                raise ValueError(f"parallel mixer: branch '{b.spec.kind}' is no projected mixer (projections, core, "
                                 f"output projection); only those can share the two products")

    @property
    def graph_safe(self):
        return all(b.graph_safe for b in self.branches)

    def cache_spec(self):
        return _kept_by(self.branches)

    def param_specs(self):
        out = {}
        for b in self.branches:
            out.update(b.param_specs())
        return out

    def load(self, get) -> None:
        self.w_in, self.b_in, self.cols = _load_and_pack_inputs(self.branches, get)
        if any(b.out_bias() is not None for b in self.branches):
            raise ValueError("parallel mixer: a bias of a branch's output projection is not built where the branches share "
                             "one output product")
        self.w_out, self.out_cols, self.k_out = pack_columns([b.out_matrix() for b in self.branches])
        self.padded = self.k_out != sum(b.inner_size() for b in self.branches)
        for b in self.branches:
            b.release_unpacked()

    def weight_bytes(self) -> int:
        return (sum(m.numel() * m.element_size() for m in (self.w_in, self.w_out, self.b_in) if m is not None)
                + sum(b.extra_weight_bytes() for b in self.branches))

    def first_product(self):
        return self.rt.ops.product_hint(self.w_in, "linear")

    def forward(self, h, ctx, cache):
        ops = self.rt.ops
        T = h.shape[0]
        y = torch.empty((T, self.w_in.shape[0]), dtype=h.dtype, device=h.device)
        ops.linear(h, self.w_in, self.b_in, y)
        act = (torch.zeros if self.padded else torch.empty)((T, self.k_out), dtype=h.dtype, device=h.device)
        views = list(cache) if isinstance(cache, (tuple, list)) else ([cache] if cache is not None else [])
        for b, cols, col, scale in zip(self.branches, self.cols, self.out_cols, self.spec.scales):
            b.core(y, cols, ctx, take_views(views, b.cache_spec()), act, col, float(scale))
        return ops.linear_to_stream(act, self.w_out, None, then=self.then)


def _kept_by(branches):
    """What the branches keep between steps, as one flat tuple in the order of the branches (None if nothing)."""
    kept = []
    for b in branches:
        spec = b.cache_spec()
        if spec is not None:
            kept += list(spec) if isinstance(spec, (tuple, list)) else [spec]
    return tuple(kept) if kept else None


def _load_and_pack_inputs(branches, get):
    """Loads the branches and packs all their input matrices (and biases) for one product: the packed matrix, the packed
    bias or None, and for every branch the first columns of its projections' results."""
    mats, biases, counts = [], [], []
    for b in branches:
        b.load(get)
        m = b.in_matrices()
        bias = b.in_biases()
        mats += m
        biases += list(bias) if bias is not None else [None] * len(m)
        counts.append(len(m))
    w_in, cols = pack_rows(mats)
    b_in = pack_biases(mats, biases)
    per_branch, at = [], 0
    for n in counts:
        per_branch.append(cols[at:at + n])
        at += n
    return w_in, b_in, per_branch


@register_part("mixer", "parallel_normed")
class NormedParallelMixer(Mixer):
    """See ``NormedParallelSpec``: every branch a ``ProjectedMixer``.  One product over all branches' input matrices (and
    biases), the cores one after the other, then each branch's own output product with its 32-bit sums left unrounded,
    and one kernel that divides each result by its root mean square, multiplies by its weight and scale and adds them,
    all in 32-bit.  The sum goes to the residual stream as it is (32-bit)."""

    def __init__(self, spec, prefix, rt):
        super().__init__(spec, prefix, rt)
        n = len(spec.branches)
        if not n or not (n == len(spec.scales) == len(spec.prefixes) == len(spec.norm_names)):
            raise ValueError("parallel_normed mixer: one scale, one prefix and one norm weight for each branch")
        if n > 4:
            raise ValueError("parallel_normed mixer: up to four branches")
        self.branches = [build_part("mixer", b, prefix + p, rt) for b, p in zip(spec.branches, spec.prefixes)]
        for b in self.branches:
            b.standalone = False
            if not isinstance(b, ProjectedMixer):
                raise ValueError(f"parallel_normed mixer: branch '{b.spec.kind}' is no projected mixer (projections, core, "
                                 f"output projection)")

    @property
    def graph_safe(self):
        return all(b.graph_safe for b in self.branches)

    def cache_spec(self):
        return _kept_by(self.branches)

    def param_specs(self):
        from .base import ParamSpec
        out = {}
        for b in self.branches:
            out.update(b.param_specs())
        for name in self.spec.norm_names:
            out[self.prefix + name] = ParamSpec((self.spec.hidden,), role="vector", init="one_plus_normal")
        return out

    def load(self, get) -> None:
        self.w_in, self.b_in, self.cols = _load_and_pack_inputs(self.branches, get)
        self.w_outs, self.b_outs, self.k_outs = [], [], []
        for b in self.branches:
            w, _, k = pack_columns([b.out_matrix()])
            self.w_outs.append(w)
            self.k_outs.append(k)
            self.b_outs.append(b.out_bias())
        self.weights = [self.rt.param(get(self.prefix + name), "vector") for name in self.spec.norm_names]
        for b in self.branches:
            b.release_unpacked()

    def weight_bytes(self) -> int:
        mats = [self.w_in, self.b_in, *self.w_outs, *self.b_outs, *self.weights]
        return (sum(m.numel() * m.element_size() for m in mats if m is not None)
                + sum(b.extra_weight_bytes() for b in self.branches))

    def first_product(self):
        return self.rt.ops.product_hint(self.w_in, "linear")

    def forward(self, h, ctx, cache):
        ops, s = self.rt.ops, self.spec
        T = h.shape[0]
        y = torch.empty((T, self.w_in.shape[0]), dtype=h.dtype, device=h.device)
        ops.linear(h, self.w_in, self.b_in, y)
        views = list(cache) if isinstance(cache, (tuple, list)) else ([cache] if cache is not None else [])
        acts = []
        for b, cols, k_out in zip(self.branches, self.cols, self.k_outs):
            act = (torch.zeros if k_out != b.inner_size() else torch.empty)((T, k_out), dtype=h.dtype, device=h.device)
            b.core(y, cols, ctx, take_views(views, b.cache_spec()), act, 0, 1.0)
            acts.append(act)
        results = []
        for act, w, bias in zip(acts, self.w_outs, self.b_outs):
            r = torch.empty((T, s.hidden), dtype=torch.float32, device=h.device)
            ops.linear(act, w, bias, r)
            results.append(r)
        total = torch.empty((T, s.hidden), dtype=torch.float32, device=h.device)
        ops.normed_sum(results, self.weights, s.eps, [float(c) for c in s.scales], total)
        # the 32-bit sum reaches the stream unrounded: as the one share of a product where the compute dtype is narrower
        return total if self.rt.dtype == torch.float32 else ops.SplitSum(total.unsqueeze(0))
