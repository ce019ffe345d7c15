"""Geponex as a ``ModelSpec``: a decoder whose layers mix tokens by softmax attention over a narrow latent a token (with
or without a sink in the softmax and an output gate) or by linear attention with a fixed decay a head over activated
projections; every mixer reads its input shifted towards the token before; the norms (root mean square in groups) come
after the residual sums, in which the stream is scaled; the feed-forward is dense with the xIELU activation and biases,
or a mixture of clamped gated experts with sigmoid scores and a shared expert; a layer may use another layer's weights
with a cache or state of its own; the output head is the embedding table.

Tensor names: ``embed``, ``final.norm``, and for layer i ``l<i>.norm1``, ``l<i>.norm2``, ``l<i>.shift``, ``l<i>.mix.*`` and
``l<i>.mlp.*``."""
from __future__ import annotations

from ..config.geponex import GeponexConfig, GeponexDense, GeponexExperts
from ..config.registry import register_architecture
from ..parts.specs import (BlockSpec, EmbeddingSpec, ExpertsSpec, HeadSpec, LatentAttentionSpec, LightningSpec, ModelSpec, NormSpec,
                           PositionSpec, RunSpec, XieluMLPSpec)


def _position(rot) -> PositionSpec:
    if not rot.dims:
        return PositionSpec(kind="none")
    sc = rot.scaling
    return PositionSpec(kind="rotary_interleaved", dim=rot.dims, base=rot.base,
                        ramp=None if sc is None else (sc.factor, sc.original, sc.fast, sc.slow))


def _block(cfg: GeponexConfig, i: int, norm: NormSpec) -> BlockSpec:
    layer = cfg.layers[i]
    m = layer.mixer
    if layer.type == "lightning":
        mixer = LightningSpec(hidden=cfg.width, heads=m.heads, dim=m.dim, v_dim=m.vdim, decay=m.decay, norm_eps=cfg.norm_eps)
    else:
        mixer = LatentAttentionSpec(hidden=cfg.width, heads=m.heads, head_dim=m.dim, rot_dim=m.rot_dim, v_dim=m.vdim, q_rank=m.q_rank,
                                    kv_rank=m.kv_rank, scale=m.scale, sink=m.second, gate=m.second, norm_eps=cfg.norm_eps,
                                    position=_position(m.rot))
    f = layer.mlp
    ffn = None
    if isinstance(f, GeponexDense):
        ffn = XieluMLPSpec(hidden=cfg.width, inter=f.ff)
    elif isinstance(f, GeponexExperts):
        ffn = ExpertsSpec(hidden=cfg.width, experts=f.experts, top=f.top, inter=f.ff, shared_inter=f.shared_ff, activation="clamped",
                          limit=f.limit, shared_limit=f.shared_limit, router_weights="sigmoid_share", router_scale=f.scale)
    return BlockSpec(mixer=mixer, ffn=ffn, norm1=norm, norm2=None if ffn is None else norm, prefix=f"l{i}.", mixer_prefix="mix.",
                     ffn_prefix="mlp.", norm1_name="norm1", norm2_name="norm2", kind="postnorm", stream_scale=cfg.postln_alpha,
                     shift_name="shift")


def geponex_model_spec(cfg: GeponexConfig) -> ModelSpec:
    norm = NormSpec(size=cfg.width, eps=cfg.norm_eps, kind="rmsnorm", weight_suffix="", groups=cfg.norm_groups)
    # a block for every layer that has tensors of its own; a layer that uses another's weights is one more run of that
    # layer's block, with cache slots of its own (the shifted row first, then what the mixer keeps)
    owners = sorted({cfg.owner(i) for i in range(len(cfg.layers))})
    block_of = {layer: n for n, layer in enumerate(owners)}
    blocks = tuple(_block(cfg, i, norm) for i in owners)
    order = tuple(RunSpec(block=block_of[cfg.owner(i)], cache=(2 * i, 2 * i + 1)) for i in range(len(cfg.layers)))
    embedding = EmbeddingSpec(vocab=cfg.vocab, hidden=cfg.width, name="embed")
    head = HeadSpec(vocab=cfg.vocab, hidden=cfg.width, norm=norm, norm_name="final.norm", name="head", tied_to="embed")
    return ModelSpec(vocab=cfg.vocab, hidden=cfg.width, blocks=blocks, order=order, embedding=embedding, head=head, max_positions=0)


register_architecture("Geponex", GeponexConfig, geponex_model_spec, replace=True)
