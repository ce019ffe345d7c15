"""Grouped-query attention over a paged cache of keys and values."""
from __future__ import annotations

import math

import torch

from .base import KVCacheSpec, Mixer, ParamSpec, build_part, register_part
from .projected import ProjectedMixer


def _attention(spec, prefix, rt):
    """The attention mixer for a spec: the kernels of ``PagedAttention`` take the whole head rotated from a table,
    values as wide as keys and a causal or windowed mask; everything else runs ``GeneralAttention``."""
    plain = (spec.v_dim in (None, spec.head_dim) and spec.qk_norm_eps is None and spec.chunk is None
             and spec.position.kind != "rotary_computed" and not spec.keep_first and spec.proj_norm_eps is None
             and spec.q_temp is None and spec.softcap is None and spec.sink == "none" and spec.gate == "none"
             and spec.weight_suffix == ".weight" and spec.bias_suffix == ".bias")
    return (PagedAttention if plain else GeneralAttention)(spec, prefix, rt)


register_part("mixer", "attention", _attention)


class PagedAttention(Mixer):
    """q, k, v = h Wq^T + bq, h Wk^T + bk, h Wv^T + bv (one product over the packed rows of
    the three matrices, which equals the three separate products of
    v1/models/qwen2-7b/inference_fp16.dag:296,302,312 element for element); q and k are
    rotated by their positions (:297,:303); k and v go into the pages (:298,:313);
    softmax(q k^T / sqrt(d)) v over the keys the token may see (:307-318); then the o
    projection (:322).  All sizes come from the spec."""

    graph_safe = True

    def __init__(self, spec, prefix, rt):
        super().__init__(spec, prefix, rt)
        if spec.position.kind != "none" and spec.position.dim != spec.head_dim:
            # the rotation kernels turn the whole head, pairs (i, i + head_dim / 2), from a table [positions, head_dim / 2, 2]
            raise ValueError(f"attention: the position encoding covers {spec.position.dim} of the head's {spec.head_dim} "
                             f"dimensions; a rotation of part of the head is not built")
        self.position = build_part("position", spec.position, prefix, rt)
        self.q_dim = spec.heads * spec.head_dim
        self.kv_dim = spec.kv_heads * spec.head_dim
        self.scale = spec.scale if spec.scale is not None else 1.0 / math.sqrt(spec.head_dim)

    def cache_spec(self):
        return KVCacheSpec(self.spec.kv_heads, self.spec.head_dim, self.spec.window)

    def param_specs(self):
        s, p = self.spec, self.prefix
        q, k, v, o = s.names
        out = {
            f"{p}{q}.weight": ParamSpec((self.q_dim, s.hidden)),
            f"{p}{k}.weight": ParamSpec((self.kv_dim, s.hidden)),
            f"{p}{v}.weight": ParamSpec((self.kv_dim, s.hidden)),
            f"{p}{o}.weight": ParamSpec((s.hidden, self.q_dim)),
        }
        if s.qkv_bias:
            out[f"{p}{q}.bias"] = ParamSpec((self.q_dim,), role="vector")
            out[f"{p}{k}.bias"] = ParamSpec((self.kv_dim,), role="vector")
            out[f"{p}{v}.bias"] = ParamSpec((self.kv_dim,), role="vector")
        if s.out_bias:
            out[f"{p}{o}.bias"] = ParamSpec((s.hidden,), role="vector")
        return out

    def load(self, get) -> None:
        s, p, rt = self.spec, self.prefix, self.rt
        q, k, v, o = s.names
        mats = [rt.param(get(f"{p}{n}.weight")) for n in (q, k, v)]
        if len({m.dtype for m in mats}) > 1:
            mats = [m.float() for m in mats]
        self.w_qkv = torch.cat(mats, dim=0).contiguous()
        del mats
        self.b_qkv = (torch.cat([rt.param(get(f"{p}{n}.bias"), "vector") for n in (q, k, v)]).contiguous()
                      if s.qkv_bias else None)
        self.w_o = rt.param(get(f"{p}{o}.weight"))
        self.b_o = rt.param(get(f"{p}{o}.bias"), "vector") if s.out_bias else None
        self.position.load(get)

    def weight_bytes(self) -> int:
        n = self.w_qkv.numel() * self.w_qkv.element_size() + self.w_o.numel() * self.w_o.element_size()
        for b in (self.b_qkv, self.b_o):
            if b is not None:
                n += b.numel() * b.element_size()
        return n

    def first_product(self):
        return self.rt.ops.product_hint(self.w_qkv, "stream")

    def forward(self, h, ctx, cache):
        s, ops = self.spec, self.rt.ops
        T = h.shape[0]
        after = ops.product_hint(self.w_o, "stream")
        if ops.single_token_step_is_one_kernel(ctx, h.dtype, s.heads, s.kv_heads, s.head_dim):
            qkv = ops.linear_to_stream(h, self.w_qkv, self.b_qkv, then=after)      # that kernel adds the shares of k itself
        else:
            qkv = torch.empty((T, self.q_dim + 2 * self.kv_dim), dtype=h.dtype, device=h.device)
            ops.linear(h, self.w_qkv, self.b_qkv, qkv, then=after)
        o = torch.empty((T, self.q_dim), dtype=h.dtype, device=h.device)
        ops.rope_attention(qkv, o, self.position.table, cache.k, cache.v, ctx, cache.block_table, s.heads, s.kv_heads,
                           s.head_dim, s.window, self.scale, store=cache.writes, status=ctx.status)
        return ops.linear_to_stream(o, self.w_o, self.b_o, then=self.then)


class GeneralAttention(ProjectedMixer):
    """Grouped-query attention with the options that ``PagedAttention``'s kernels do not take: values of another size
    than keys (``v_dim``), a rotation of the first dimensions of a head only, with the angle formed where it is used
    (``rotary_computed``), q and k divided by their root mean square after the rotation (``qk_norm_eps``), and a mask
    of chunks (``chunk``) beside or instead of the window; a norm of q and of k over all their heads together with a
    weight, before the rotation (``proj_norm_eps``); a query temperature that grows with the position (``q_temp``); capped
    scores (``softcap``); a sink in the softmax's denominator (``sink``); a gate on the heads' results, one number a head
    or one an element, whose matrix joins the packed input product (``gate``); biases.  One kernel norms, rotates and
    scales q and k (32-bit) and stores k and v into the pages; the attention kernel walks the visible keys of every
    (token, head) with a running maximum and sum in 32-bit and ends with the sink and the gate."""

    def __init__(self, spec, prefix, rt):
        super().__init__(spec, prefix, rt)
        if spec.sink not in ("none", "zero", "learned"):
            raise ValueError(f"attention: sink '{spec.sink}' is not known; known: none, zero, learned")
        if spec.gate not in ("none", "head", "element"):
            raise ValueError(f"attention: gate '{spec.gate}' is not known; known: none, head, element")
        if spec.proj_norm_eps is not None and spec.qk_norm_eps is not None:
            raise ValueError("attention: a norm of q and k over the whole projection or head by head, not both")
        if spec.position.kind not in ("rotary_computed", "none"):
            raise ValueError(f"attention: position encoding '{spec.position.kind}' is not built beside the general options; "
                             f"known: rotary_computed, none")
        if spec.position.kind != "none" and (spec.position.dim % 2 or spec.position.dim > spec.head_dim):
            raise ValueError(f"attention: the rotation covers {spec.position.dim} dimensions; it must be even and at most "
                             f"the head's {spec.head_dim}")
        self.position = build_part("position", spec.position, prefix, rt)
        self.v_dim = spec.v_dim if spec.v_dim else spec.head_dim
        self.scale = spec.scale if spec.scale is not None else 1.0 / math.sqrt(spec.head_dim)

    def cache_spec(self):
        s = self.spec
        return KVCacheSpec(s.kv_heads, s.head_dim, s.window, v_dim=self.v_dim if self.v_dim != s.head_dim else None,
                           keep_first=s.keep_first if s.window else 0)

    def param_specs(self):
        s, p, x, bx = self.spec, self.prefix, self.spec.weight_suffix, self.spec.bias_suffix
        q, k, v, o = s.names
        sizes = {q: s.heads * s.head_dim, k: s.kv_heads * s.head_dim, v: s.kv_heads * self.v_dim}
        out = {f"{p}{n}{x}": ParamSpec((size, s.hidden)) for n, size in sizes.items()}
        out[f"{p}{o}{x}"] = ParamSpec((s.hidden, s.heads * self.v_dim))
        if s.qkv_bias:
            out.update({f"{p}{n}{bx}": ParamSpec((size,), role="vector") for n, size in sizes.items()})
        if s.out_bias:
            out[f"{p}{o}{bx}"] = ParamSpec((s.hidden,), role="vector")
        if s.proj_norm_eps is not None:
            out[p + s.norm_names[0]] = ParamSpec((sizes[q],), role="vector", init="one_plus_normal")
            out[p + s.norm_names[1]] = ParamSpec((sizes[k],), role="vector", init="one_plus_normal")
        if s.sink == "learned":
            out[p + s.sink_name] = ParamSpec((s.heads,), role="vector")
        if s.gate != "none":
            out[p + s.gate_name] = ParamSpec((s.heads if s.gate == "head" else s.heads * self.v_dim, s.hidden))
        return out

    def load(self, get) -> None:
        s, p, rt, x, bx = self.spec, self.prefix, self.rt, self.spec.weight_suffix, self.spec.bias_suffix
        q, k, v, o = s.names
        self._in = [rt.param(get(f"{p}{n}{x}")) for n in (q, k, v)]
        self._in_bias = [rt.param(get(f"{p}{n}{bx}"), "vector") for n in (q, k, v)] if s.qkv_bias else [None, None, None]
        if s.gate != "none":
            self._in.append(rt.param(get(p + s.gate_name)))
            self._in_bias.append(None)
        self.w_o = rt.param(get(f"{p}{o}{x}"))
        self.b_o = rt.param(get(f"{p}{o}{bx}"), "vector") if s.out_bias else None
        self.q_weight = self.k_weight = None
        if s.proj_norm_eps is not None:
            self.q_weight = rt.param(get(p + s.norm_names[0]), "vector")
            self.k_weight = rt.param(get(p + s.norm_names[1]), "vector")
        self.sinks = None
        if s.sink == "learned":
            self.sinks = rt.param(get(p + s.sink_name), "vector")
        elif s.sink == "zero":
            self.sinks = torch.zeros(s.heads, dtype=torch.float32, device=rt.device)
        self.position.load(get)
        self.pack()

    def release_unpacked(self) -> None:
        self._in = self.w_o = None

    def in_matrices(self):
        return list(self._in)

    def in_biases(self):
        return list(self._in_bias) if any(b is not None for b in self._in_bias) else None

    def out_matrix(self):
        return self.w_o

    def out_bias(self):
        return self.b_o

    def inner_size(self) -> int:
        return self.spec.heads * self.v_dim

    def extra_weight_bytes(self) -> int:
        return sum(4 * t.numel() for t in (self.q_weight, self.k_weight, self.sinks) if t is not None)

    def core(self, y, cols, ctx, cache, out, out_col, out_scale) -> None:
        s, ops = self.spec, self.rt.ops
        freq = getattr(self.position, "frequencies", None)
        k_pages, v_pages = cache.pages["k"], cache.pages["v"]
        whole = s.proj_norm_eps is not None
        ops.attention_prepare(y, cols[0], cols[1], cols[2], ctx, freq, s.proj_norm_eps if whole else s.qk_norm_eps, k_pages, v_pages,
                              cache.block_table, s.heads, s.kv_heads, s.head_dim, self.v_dim, store=cache.writes, status=ctx.status,
                              q_weight=self.q_weight, k_weight=self.k_weight, norm_first=whole, whole_projection=whole,
                              rot_mult=getattr(self.position, "mult", 1.0), q_temp=s.q_temp)
        gated = s.gate != "none"
        extras = s.softcap is not None or self.sinks is not None
        takes = ops.tensor_core_attention_takes_extras if extras else ops.tensor_core_attention_takes
        if cols[0] == 0 and not s.keep_first and takes(y.dtype, s.heads, s.kv_heads, s.head_dim, self.v_dim, cache.page_size):
            # values as wide as keys at a head size the tensor-core kernels take: the kernels of the plain attention walk
            # the keys (tcgen05 for long portions, mma.sync tiles, the single-token kernel; the mma.sync kernel where there
            # is a sink or a cap), with the chunks as one more bound of the keys a row sees.  They write a tensor of their
            # own, which is then gated and scaled into its columns.
            n = s.heads * self.v_dim
            direct = out_col == 0 and out.shape[1] == n and out_scale == 1.0 and not gated
            o = out if direct else torch.empty((y.shape[0], n), dtype=y.dtype, device=y.device)
            ops.paged_attention(y, o, k_pages, v_pages, ctx, cache.block_table, s.heads, s.kv_heads, s.head_dim, s.window,
                                self.scale, status=ctx.status, chunk=s.chunk, sinks=self.sinks, softcap=s.softcap)
            if gated:
                ops.gate_into(o, y, cols[3], s.gate, out, out_col, out_scale, s.heads, self.v_dim)
            elif not direct:
                ops.scale_into(o, out, out_col, out_scale)
            return
        ops.attention_general(y, cols[0], out, out_col, out_scale, k_pages, v_pages, ctx, cache.block_table, s.heads,
                              s.kv_heads, s.head_dim, self.v_dim, s.window, s.chunk, self.scale, status=ctx.status,
                              keep_first=s.keep_first if s.window else 0, sinks=self.sinks, softcap=s.softcap,
                              gate=s.gate, gate_col=cols[3] if s.gate != "none" else 0)


@register_part("mixer", "differential_attention")
class DifferentialAttention(ProjectedMixer):
    """See ``DifferentialAttentionSpec``.  q, k and v are one product.  One kernel norms q and k map by map (32-bit,
    weights), rotates them and stores k and v into the pages: the two maps of a head of values are two heads of keys
    ([pages, kv_heads * 2, page, head_dim]) beside one head of values.  The attention kernel walks a token's visible
    keys once for both maps (the first tokens that stay visible, then the window), each with a running maximum and sum
    of its own over the same values, and ends with the difference, its norm and the factor 1 - diff.  lam is one
    number a layer, formed in 32-bit when the weights are loaded."""

    def __init__(self, spec, prefix, rt):
        super().__init__(spec, prefix, rt)
        if spec.heads % spec.kv_heads:
            raise ValueError(f"differential attention: {spec.heads} heads over {spec.kv_heads} key/value heads")
        if spec.position.kind not in ("rotary_computed", "none"):
            raise ValueError(f"differential attention: position encoding '{spec.position.kind}' is not built; known: "
                             f"rotary_computed, none")
        if spec.position.kind != "none" and (spec.position.dim % 2 or spec.position.dim > spec.head_dim):
            raise ValueError(f"differential attention: the rotation covers {spec.position.dim} dimensions; it must be even "
                             f"and at most the head's {spec.head_dim}")
        self.position = build_part("position", spec.position, prefix, rt)
        self.scale = spec.scale if spec.scale is not None else 1.0 / math.sqrt(spec.head_dim)
        self.keep_first = spec.keep_first if spec.window else 0

    def cache_spec(self):
        s = self.spec
        return KVCacheSpec(s.kv_heads, s.head_dim, s.window, v_dim=s.v_dim if s.v_dim != s.head_dim else None, k_maps=2,
                           keep_first=self.keep_first)

    def param_specs(self):
        s, p = self.spec, self.prefix
        q, k, v, o, qn, kn, lq1, lk1, lq2, lk2 = s.names
        out = {
            p + q: ParamSpec((s.heads * 2 * s.head_dim, s.hidden)), p + k: ParamSpec((s.kv_heads * 2 * s.head_dim, s.hidden)),
            p + v: ParamSpec((s.kv_heads * s.v_dim, s.hidden)), p + o: ParamSpec((s.hidden, s.heads * s.v_dim)),
            p + qn: ParamSpec((s.head_dim,), role="vector", init="one_plus_normal"),
            p + kn: ParamSpec((s.head_dim,), role="vector", init="one_plus_normal"),
        }
        out.update({p + n: ParamSpec((s.head_dim,), role="vector") for n in (lq1, lk1, lq2, lk2)})
        return out

    def load(self, get) -> None:
        s, p, rt = self.spec, self.prefix, self.rt
        q, k, v, o, qn, kn, lq1, lk1, lq2, lk2 = s.names
        self._in = [rt.param(get(p + n)) for n in (q, k, v)]
        self.w_o = rt.param(get(p + o))
        self.q_weight = rt.param(get(p + qn), "vector")
        self.k_weight = rt.param(get(p + kn), "vector")
        l1 = float((rt.param(get(p + lq1), "vector").double() * rt.param(get(p + lk1), "vector").double()).sum())
        l2 = float((rt.param(get(p + lq2), "vector").double() * rt.param(get(p + lk2), "vector").double()).sum())
        self.lam = math.exp(l1) - math.exp(l2) + s.diff           # one number a layer, formed once
        self.position.load(get)
        self.pack()

    def release_unpacked(self) -> None:
        self._in = self.w_o = None

    def in_matrices(self):
        return list(self._in)

    def out_matrix(self):
        return self.w_o

    def inner_size(self) -> int:
        return self.spec.heads * self.spec.v_dim

    def extra_weight_bytes(self) -> int:
        return 4 * (self.q_weight.numel() + self.k_weight.numel())

    def core(self, y, cols, ctx, cache, out, out_col, out_scale) -> None:
        s, ops = self.spec, self.rt.ops
        freq = getattr(self.position, "frequencies", None)
        k_pages, v_pages = cache.pages["k"], cache.pages["v"]
        ops.attention_prepare(y, cols[0], cols[1], cols[2], ctx, freq, s.norm_eps, k_pages, v_pages, cache.block_table,
                              s.heads * 2, s.kv_heads * 2, s.head_dim, s.v_dim, store=cache.writes, status=ctx.status,
                              v_heads=s.kv_heads, q_weight=self.q_weight, k_weight=self.k_weight, norm_first=True)
        ops.attention_differential(y, cols[0], out, out_col, out_scale * (1.0 - s.diff), k_pages, v_pages, ctx, cache.block_table,
                                   s.heads, s.kv_heads, s.head_dim, s.v_dim, s.window, self.keep_first, self.scale, self.lam,
                                   s.norm_eps, status=ctx.status)
