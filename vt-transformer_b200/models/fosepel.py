"""Fosepel as a ``ModelSpec``: a decoder whose layers mix tokens by a softmax attention with a partial rotation and an
element-wise gate, or by two mixers side by side whose results are normed and averaged: a softmax attention with a sink
beside the delta rule with one decay a head, or a softmax attention with capped scores, a query temperature and a learned
sink beside a matrix memory with exponential gates.  A norm before and after each sublayer, a dense gated feed-forward, a
span of layers that may run several times with the same weights (each pass with a cache and state of its own, the
embedding's output added again before every pass but the first), and the embedding table once more as the output, with
capped logits.

Tensor names: ``embed``, ``final.norm``, and for layer i ``l<i>.norm1``, ``l<i>.norm1b``, ``l<i>.norm2``, ``l<i>.norm2b``,
``l<i>.mix.*`` (``l<i>.mix.left.*``, ``l<i>.mix.right.*``) and ``l<i>.mlp.gate|up|down``."""
from __future__ import annotations

from ..config.fosepel import FosepelAttention, FosepelConfig, FosepelDelta
from ..config.registry import register_architecture
from ..parts.specs import (AttentionSpec, BlockSpec, EmbeddingSpec, GatedDeltaSpec, GatedMLPSpec, HeadSpec, MatrixMemorySpec,
                           ModelSpec, NormedParallelSpec, NormSpec, PositionSpec, RunSpec)


def _attention(cfg: FosepelConfig, a: FosepelAttention) -> AttentionSpec:
    common = dict(hidden=cfg.width, heads=a.heads, kv_heads=a.kv_heads, head_dim=a.dim, v_dim=a.vdim, scale=a.scale,
                  names=("q", "k", "v", "o"), weight_suffix="", bias_suffix=".b")
    if a.flavour == "rotary":
        position = PositionSpec(kind="none")
        if a.rot is not None:
            sc = a.rot.scaling
            position = PositionSpec(kind="rotary_computed", dim=a.rot.dims, base=a.rot.base,
                                    ramp=None if sc is None else (sc.factor, sc.original, sc.fast, sc.slow))
        return AttentionSpec(qkv_bias=False, out_bias=False, position=position, proj_norm_eps=cfg.norm_eps, gate="element", **common)
    if a.flavour == "unit_sink":
        return AttentionSpec(qkv_bias=True, out_bias=False, proj_norm_eps=cfg.norm_eps, sink="zero", gate="head", **common)
    return AttentionSpec(qkv_bias=True, out_bias=True, sink="learned", softcap=a.softcap,
                         q_temp=None if a.q_temp_coef is None else (a.q_temp_coef, a.q_temp_every), **common)


def fosepel_model_spec(cfg: FosepelConfig) -> ModelSpec:
    norm = NormSpec(size=cfg.width, eps=cfg.norm_eps, kind="rmsnorm", weight_suffix="")
    blocks = []
    for i, layer in enumerate(cfg.layers):
        mixer = _attention(cfg, layer.left)
        if layer.right is not None:
            m = layer.right
            if isinstance(m, FosepelDelta):
                right = GatedDeltaSpec(hidden=cfg.width, heads=m.heads, kv_heads=m.kv_heads, dim=m.dim, v_dim=m.vdim, taps=m.conv,
                                       key_eps=1e-6, norm_eps=cfg.norm_eps)
            else:
                right = MatrixMemorySpec(hidden=cfg.width, heads=m.heads, dim=m.dim, v_dim=m.vdim, gate_cap=m.gate_cap,
                                         den_eps=1e-6, norm_eps=cfg.norm_eps)
            mixer = NormedParallelSpec(hidden=cfg.width, branches=(mixer, right), scales=(0.5, 0.5), prefixes=("left.", "right."),
                                       norm_names=("left.out", "right.out"), eps=cfg.norm_eps)
        ffn = None if layer.ff is None else GatedMLPSpec(hidden=cfg.width, inter=layer.ff, names=("gate", "up", "down"),
                                                         weight_suffix="")
        blocks.append(BlockSpec(mixer=mixer, ffn=ffn, norm1=norm, norm2=None if ffn is None else norm, prefix=f"l{i}.",
                                mixer_prefix="mix.", ffn_prefix="mlp.", norm1_name="norm1", norm2_name="norm2", kind="sandwich",
                                post1=norm, post2=None if ffn is None else norm, post1_name="norm1b", post2_name="norm2b"))
    # every run of a layer keeps what it keeps in slots of its own: a layer of a repeated span has keys and state for each pass
    # (an attention keeps pages; the delta rule a state and, with more than one tap, its convolutions' last inputs; the
    # matrix memory a state)
    order, slot = [], 0
    kept = [1 + (0 if l.right is None else (2 if isinstance(l.right, FosepelDelta) and l.right.conv > 1 else 1)) for l in cfg.layers]
    for b, again in cfg.run_order():
        n = kept[b]
        cache, slot = (slot if n == 1 else tuple(range(slot, slot + n))), slot + n
        order.append(RunSpec(block=b, cache=cache, add_embedding=again))
    embedding = EmbeddingSpec(vocab=cfg.vocab, hidden=cfg.width, name="embed")
    head = HeadSpec(vocab=cfg.vocab, hidden=cfg.width, norm=norm, norm_name="final.norm", name="head", tied_to="embed",
                    logit_cap=cfg.logit_softcap)
    return ModelSpec(vocab=cfg.vocab, hidden=cfg.width, blocks=tuple(blocks), order=tuple(order), embedding=embedding, head=head,
                     max_positions=0)


register_architecture("Fosepel", FosepelConfig, fosepel_model_spec, replace=True)
