"""Configuration of the Geponex decoder ("Geponex").

Its config.json is nested: ``layers`` lists the layers one by one, each with the ``type`` of its mixer
("latent_attention": softmax attention over a narrow latent a token; "latent_attention_2": the same with a sink in the
softmax's denominator and an output gate; "lightning": linear attention with one fixed decay a head over activated
projections), the mixer's sizes and constants under ``mixer``, and its feed-forward under ``mlp`` (dense, a mixture of
experts, or null).  A layer with ``weights_of``: j has no tensors of its own and uses layer j's, with a cache or state
of its own.  The norms come after the residual sums (``postln_alpha`` scales the stream in the sum) and cut the vector
into ``norm.groups`` parts.  Every size and every constant that can differ between two models of the design is read
from there.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Optional, Tuple

from .base import ConfigError, KeyReader, ModelConfig, architecture_name


@dataclass(frozen=True)
class RotationRamp:
    """Frequencies blended towards f / ``factor`` by a ramp over the pair index between the pairs that turn ``fast`` and
    ``slow`` times within ``original`` positions."""
    factor: float
    original: float
    fast: float
    slow: float


@dataclass(frozen=True)
class GeponexRotation:
    dims: int
    base: float
    scaling: Optional[RotationRamp] = None


@dataclass(frozen=True)
class GeponexLatentAttention:
    """``heads`` heads with ``dim`` plain and ``rot_dim`` rotated query/key dimensions and values of ``vdim``; queries
    through a latent of ``q_rank``, keys and values from a latent of ``kv_rank``.  ``second``: the variant with a sink
    and an output gate."""
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    q_rank: int
    kv_rank: int
    scale: float
    rot: GeponexRotation
    second: bool


@dataclass(frozen=True)
class GeponexLightning:
    heads: int
    dim: int
    vdim: int
    decay: Tuple[float, ...]


@dataclass(frozen=True)
class GeponexDense:
    ff: int


@dataclass(frozen=True)
class GeponexExperts:
    """``experts`` clamped gated feed-forwards of inner size ``ff`` of which a token uses ``top``, weighted by their
    sigmoid scores over the chosen ones' sum, times ``scale``; ``shared_ff``: the inner size of the expert every token
    uses (None: there is none), with a clamp of its own."""
    experts: int
    top: int
    scale: float
    ff: int
    limit: float
    shared_ff: Optional[int]
    shared_limit: float


@dataclass(frozen=True)
class GeponexLayer:
    type: str
    mixer: Any                          # GeponexLatentAttention or GeponexLightning
    mlp: Any                            # GeponexDense, GeponexExperts or None
    weights_of: Optional[int] = None


@dataclass(frozen=True)
class GeponexConfig(ModelConfig):
    vocab: int
    width: int
    layers: Tuple[GeponexLayer, ...]
    norm_eps: float
    norm_groups: int
    postln_alpha: float

    def owner(self, i: int) -> int:
        """The layer whose tensors layer i uses."""
        seen = set()
        while self.layers[i].weights_of is not None:
            if i in seen:
                raise ConfigError(f"layers[{i}]: 'weights_of' runs in a circle")
            seen.add(i)
            i = self.layers[i].weights_of
        return i

    # ---- reading -------------------------------------------------------------------
    @classmethod
    def from_dict(cls, data: Dict[str, Any], where: str = "config.json") -> "GeponexConfig":
        r = KeyReader(data, where)
        arch = architecture_name(data, where)
        layers_raw = r.raw("layers")
        if not isinstance(layers_raw, list) or not layers_raw:
            raise ConfigError(f"{where}: key 'layers' must be a list with one entry for each layer")
        layers = tuple(_layer(entry, f"{where}: layers[{i}]") for i, entry in enumerate(layers_raw))
        norm = KeyReader(_obj(r.raw("norm"), f"{where}: norm"), f"{where}: norm")
        cfg = cls(architecture=arch, vocab=r.integer("vocab", minimum=1), width=r.integer("width", minimum=1), layers=layers,
                  norm_eps=norm.number("eps", positive=True), norm_groups=norm.integer("groups", default=1, minimum=1),
                  postln_alpha=r.number("postln_alpha", default=1.0))
        cfg.validate(where)
        return cfg

    def validate(self, where: str = "config.json") -> None:
        if self.width % 8:
            raise ConfigError(f"{where}: 'width' {self.width} is not supported: the matrix kernels read rows in "
                              f"16-byte pieces, so it must be a multiple of 8")
        if self.width % self.norm_groups:
            raise ConfigError(f"{where}: norm 'groups' {self.norm_groups} must cut 'width' {self.width} into equal parts")
        for i, layer in enumerate(self.layers):
            at = f"{where}: layers[{i}]"
            if layer.weights_of is not None:
                j = layer.weights_of
                if not 0 <= j < len(self.layers) or j == i:
                    raise ConfigError(f"{at}: 'weights_of' {j} names no other layer")
                o = self.layers[self.owner(i)]
                if o.type != layer.type:
                    raise ConfigError(f"{at}: 'weights_of' {j} names a layer of another type ('{o.type}'); the sizes and "
                                      f"constants are taken from the layer that owns the weights")
            m = layer.mixer
            if layer.type == "lightning":
                if len(m.decay) != m.heads:
                    raise ConfigError(f"{at}: 'decay' lists {len(m.decay)} numbers for {m.heads} heads")
                if m.dim > 1024:
                    raise ConfigError(f"{at}: 'dim' above 1024 is not supported by the scan kernel")
            else:
                if m.rot.dims % 2 or m.rot.dims > m.rot_dim:
                    raise ConfigError(f"{at}: 'rot.dims' {m.rot.dims} must be even and at most 'rot_dim' {m.rot_dim}")
                if m.kv_rank + m.rot_dim > 2048 or m.kv_rank > 1024:
                    raise ConfigError(f"{at}: 'kv_rank' above 1024 (or with 'rot_dim' above 2048) is not supported by the "
                                      f"attention kernel")
                if max(m.dim, m.kv_rank) > 1536:
                    raise ConfigError(f"{at}: 'dim' above 1536 is not supported by the heads' products")
            f = layer.mlp
            if isinstance(f, GeponexExperts):
                if not 1 <= f.top <= f.experts:
                    raise ConfigError(f"{at}: router 'top' {f.top} must lie between 1 and 'experts' {f.experts}")
                if f.experts > 1024:
                    raise ConfigError(f"{at}: more than 1024 experts are not supported by the routing kernel")

    def to_dict(self) -> Dict[str, Any]:
        return {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
                "layers": [_layer_dict(layer) for layer in self.layers],
                "norm": {"eps": self.norm_eps, "groups": self.norm_groups}, "postln_alpha": self.postln_alpha}


def _obj(v, where: str) -> Dict[str, Any]:
    if not isinstance(v, dict):
        raise ConfigError(f"{where}: expected an object")
    return v


def _rotation(raw, where: str, default_dims: int) -> GeponexRotation:
    if raw is None:
        return GeponexRotation(dims=0, base=10000.0)
    r = KeyReader(_obj(raw, where), where)
    scaling = None
    sc = r.raw("scaling", default=None)
    if sc is not None:
        s = KeyReader(_obj(sc, where + ".scaling"), where + ".scaling")
        scaling = RotationRamp(factor=s.number("factor", positive=True), original=s.number("original", positive=True),
                               fast=s.number("fast", positive=True), slow=s.number("slow", positive=True))
    return GeponexRotation(dims=r.integer("dims", default=default_dims, minimum=0), base=r.number("base", positive=True),
                           scaling=scaling)


def _layer(entry, where: str) -> GeponexLayer:
    r = KeyReader(_obj(entry, where), where)
    kind = r.string("type")
    mw = f"{where}.mixer"
    m = KeyReader(_obj(r.raw("mixer"), mw), mw)
    if kind in ("latent_attention", "latent_attention_2"):
        dim, rot_dim = m.integer("dim", minimum=1), m.integer("rot_dim", minimum=0)
        mixer = GeponexLatentAttention(heads=m.integer("heads", minimum=1), dim=dim, rot_dim=rot_dim,
                                       vdim=m.integer("vdim", default=dim, minimum=1), q_rank=m.integer("q_rank", minimum=1),
                                       kv_rank=m.integer("kv_rank", minimum=1),
                                       scale=m.number("scale", default=(dim + rot_dim) ** -0.5),
                                       rot=_rotation(m.raw("rot", default=None), mw + ".rot", rot_dim),
                                       second=kind == "latent_attention_2")
    elif kind == "lightning":
        decay = m.raw("decay")
        if isinstance(decay, (int, float)) and not isinstance(decay, bool):      # one number for all heads
            decay = [decay] * m.integer("heads", minimum=1)
        if not isinstance(decay, list) or not all(isinstance(d, (int, float)) and not isinstance(d, bool) for d in decay):
            raise ConfigError(f"{mw}: key 'decay' must be a list of numbers, one for each head")
        dim = m.integer("dim", minimum=1)
        mixer = GeponexLightning(heads=m.integer("heads", minimum=1), dim=dim, vdim=m.integer("vdim", default=dim, minimum=1),
                                 decay=tuple(float(d) for d in decay))
    else:
        raise ConfigError(f"{where}: layer type '{kind}' is not known; known are 'latent_attention', 'latent_attention_2' "
                          f"and 'lightning'")
    mlp_raw = r.raw("mlp", default=None)
    mlp = None
    if mlp_raw is not None:
        fw = f"{where}.mlp"
        f = KeyReader(_obj(mlp_raw, fw), fw)
        ff_kind = f.string("kind")
        if ff_kind == "dense":
            mlp = GeponexDense(ff=f.integer("ff", minimum=1))
        elif ff_kind == "moe":
            router = KeyReader(_obj(f.raw("router"), fw + ".router"), fw + ".router")
            exp = KeyReader(_obj(f.raw("expert"), fw + ".expert"), fw + ".expert")
            shared_raw = f.raw("shared", default=None)
            shared_ff, shared_limit = None, 0.0
            if shared_raw is not None:
                sh = KeyReader(_obj(shared_raw, fw + ".shared"), fw + ".shared")
                shared_ff, shared_limit = sh.integer("ff", minimum=1), sh.number("limit", positive=True)
            mlp = GeponexExperts(experts=router.integer("experts", minimum=1), top=router.integer("top", minimum=1),
                                 scale=router.number("scale", default=1.0), ff=exp.integer("ff", minimum=1),
                                 limit=exp.number("limit", positive=True), shared_ff=shared_ff, shared_limit=shared_limit)
        else:
            raise ConfigError(f"{fw}: feed-forward kind '{ff_kind}' is not known; known are 'dense' and 'moe'")
    return GeponexLayer(type=kind, mixer=mixer, mlp=mlp, weights_of=r.integer("weights_of", default=None, minimum=0))


def _layer_dict(layer: GeponexLayer) -> Dict[str, Any]:
    m = layer.mixer
    if layer.type == "lightning":
        mixer = {"heads": m.heads, "dim": m.dim, "vdim": m.vdim, "decay": list(m.decay)}
    else:
        rot = {"dims": m.rot.dims, "base": m.rot.base}
        if m.rot.scaling is not None:
            s = m.rot.scaling
            rot["scaling"] = {"factor": s.factor, "original": s.original, "fast": s.fast, "slow": s.slow}
        mixer = {"heads": m.heads, "dim": m.dim, "rot_dim": m.rot_dim, "vdim": m.vdim, "q_rank": m.q_rank, "kv_rank": m.kv_rank,
                 "scale": m.scale, "rot": rot}
    f = layer.mlp
    mlp = None
    if isinstance(f, GeponexDense):
        mlp = {"kind": "dense", "ff": f.ff}
    elif isinstance(f, GeponexExperts):
        mlp = {"kind": "moe", "router": {"experts": f.experts, "top": f.top, "scale": f.scale},
               "expert": {"ff": f.ff, "limit": f.limit},
               "shared": None if f.shared_ff is None else {"ff": f.shared_ff, "limit": f.shared_limit}}
    out = {"type": layer.type, "mixer": mixer, "mlp": mlp}
    if layer.weights_of is not None:
        out["weights_of"] = layer.weights_of
    return out
