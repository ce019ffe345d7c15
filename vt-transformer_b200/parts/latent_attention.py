"""Softmax attention over a narrow latent that is all a token keeps."""
from __future__ import annotations

import torch

from .base import LatentCacheSpec, ParamSpec, build_part, register_part
from .projected import ProjectedMixer, _round_up, pack_rows


@register_part("mixer", "latent_attention")
class LatentAttention(ProjectedMixer):
    """See ``LatentAttentionSpec``.  A token keeps its normed latent c and the rotated key part r that the heads share,
    side by side in one row of a page.  Head i's key is [U_i c | r] and its value V_i c, so with q = [q_u | q_r]:
    q . k = (U_i^T q_u) . c + q_r . r, and sum_j p_j V_i c_j = V_i sum_j p_j c_j.  The step therefore takes the queries
    into the latent's space once a token (a product of each head with its own U_i^T, which also rotates q_r), runs one
    attention in which every head reads the same rows (a value is the first ``kv_rank`` numbers of its key's row), and
    takes each head's result through V_i; keys and values of single heads are never formed.  D_q, D_kv and the gate's
    matrix are one product; one kernel norms both latents, rotates r and stores the row."""

    def __init__(self, spec, prefix, rt):
        super().__init__(spec, prefix, rt)
        pos = spec.position
        if pos.kind not in ("rotary_interleaved", "none"):
            raise ValueError(f"latent attention: position encoding '{pos.kind}' is not built; known: rotary_interleaved, none")
        if pos.kind != "none" and (pos.dim % 2 or pos.dim > spec.rot_dim):
            raise ValueError(f"latent attention: the rotation covers {pos.dim} dimensions; it must be even and at most the "
                             f"rotated part's {spec.rot_dim}")
        self.position = build_part("position", pos, prefix, rt)
        self.q_head = spec.head_dim + spec.rot_dim            # a head's query as the up projection leaves it
        self.key = spec.kv_rank + spec.rot_dim                # a token's row, and a head's query in the latent's space

    def cache_spec(self):
        return LatentCacheSpec(self.key)

    def param_specs(self):
        s, p = self.spec, self.prefix
        dq, dqn, uq, dkv, dkvn, uk, uv, o, sink, g = s.names
        out = {
            p + dq: ParamSpec((s.q_rank, s.hidden)), p + dqn: ParamSpec((s.q_rank,), role="vector", init="one_plus_normal"),
            p + uq: ParamSpec((s.heads * self.q_head, s.q_rank)), p + dkv: ParamSpec((self.key, s.hidden)),
            p + dkvn: ParamSpec((s.kv_rank,), role="vector", init="one_plus_normal"),
            p + uk: ParamSpec((s.heads * s.head_dim, s.kv_rank)), p + uv: ParamSpec((s.heads * s.v_dim, s.kv_rank)),
            p + o: ParamSpec((s.hidden, s.heads * s.v_dim)),
        }
        if s.sink:
            out[p + sink] = ParamSpec((s.heads,), role="vector")
        if s.gate:
            out[p + g] = ParamSpec((s.heads * s.v_dim, s.hidden))
        return out

    def load(self, get) -> None:
        s, p, rt = self.spec, self.prefix, self.rt
        dq, dqn, uq, dkv, dkvn, uk, uv, o, sink, g = s.names
        self._in = [rt.param(get(p + n)) for n in ((dq, dkv, g) if s.gate else (dq, dkv))]
        self.w_o = rt.param(get(p + o))
        self.q_weight = rt.param(get(p + dqn), "vector")
        self.k_weight = rt.param(get(p + dkvn), "vector")
        # the queries' up projection reads the normed latent in a buffer whose rows are padded to 16 bytes
        self.q_rank_p = _round_up(s.q_rank)
        w_uq = rt.param(get(p + uq))
        if self.q_rank_p != s.q_rank:
            w_uq = torch.cat([w_uq, torch.zeros((w_uq.shape[0], self.q_rank_p - s.q_rank), dtype=w_uq.dtype, device=w_uq.device)], dim=1)
        self.w_uq, _ = pack_rows([w_uq])        # rows padded to a multiple of 8
        # U [heads, head_dim, kv_rank] takes a head's plain query part into the latent's space; V [heads, kv_rank, v_dim]
        # takes a head's result out of it
        self.u = rt.param(get(p + uk)).view(s.heads, s.head_dim, s.kv_rank).contiguous()
        self.v = rt.param(get(p + uv)).view(s.heads, s.v_dim, s.kv_rank).transpose(1, 2).contiguous()
        self.sinks = rt.param(get(p + sink), "vector") if s.sink else None
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
        small = [self.w_uq, self.u, self.v, self.q_weight, self.k_weight] + ([self.sinks] if self.sinks is not None else [])
        return sum(t.numel() * t.element_size() for t in small)

    def core(self, y, cols, ctx, cache, out, out_col, out_scale) -> None:
        s, ops = self.spec, self.rt.ops
        T, dev = y.shape[0], y.device
        freq, mult = self.position.frequencies if s.position.kind != "none" else None, getattr(self.position, "mult", 1.0)
        pages = cache.pages["c"]
        padded = self.q_rank_p != s.q_rank
        cq = (torch.zeros if padded else torch.empty)((T, self.q_rank_p), dtype=y.dtype, device=dev)
        ops.latent_prepare(y, cols[0], s.q_rank, cols[1], s.kv_rank, s.rot_dim, self.q_weight, self.k_weight, s.norm_eps, freq, mult,
                           ctx, cache.block_table, cq, pages, store=cache.writes, status=ctx.status)
        q = torch.empty((T, self.w_uq.shape[0]), dtype=y.dtype, device=dev)
        ops.linear(cq, self.w_uq, None, q)
        qa = torch.empty((T, s.heads * self.key), dtype=y.dtype, device=dev)
        ops.head_matmul(q, 0, self.q_head, self.u, qa, 0, self.key, mode="rotated_tail", tail=s.rot_dim, frequencies=freq, mult=mult,
                        ctx=ctx)
        oc = torch.empty((T, s.heads * s.kv_rank), dtype=y.dtype, device=dev)
        ops.attention_latent(qa, 0, oc, 0, pages, ctx, cache.block_table, s.heads, self.key, s.kv_rank, s.scale, sinks=self.sinks,
                             status=ctx.status)
        direct = out_scale == 1.0
        o = out if direct else torch.empty((T, s.heads * s.v_dim), dtype=y.dtype, device=dev)
        ops.head_matmul(oc, 0, s.kv_rank, self.v, o, out_col if direct else 0, s.v_dim, mode="gate" if s.gate else "plain",
                        gate=y if s.gate else None, gate_col=cols[2] if s.gate else 0)
        if not direct:
            ops.scale_into(o, out, out_col, out_scale)
