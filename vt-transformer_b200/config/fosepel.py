"""Configuration of the Fosepel decoder ("Fosepel").

Its config.json is nested: ``layers`` lists the layers one by one, each with the ``type`` of its mixer ("attention":
softmax attention with a partial rotation and a gate; "parallel": a softmax attention with a sink beside the delta rule
with one decay a head; "parallel_2": a softmax attention with capped scores and a learned sink beside a matrix memory
with exponential gates), the mixer's sizes and constants under ``mixer`` (for the two parallel types under ``left`` and
``right``), and its feed-forward under ``mlp`` (dense, or null).  ``loop`` names a span of layers that runs several
times in a row with the same weights.  Every size and every constant that can differ between two models of the design
is read from there.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Optional, Tuple

from .base import ConfigError, KeyReader, ModelConfig, architecture_name


@dataclass(frozen=True)
class FosepelRamp:
    """The blend of the rotation's frequencies between the pairs that turn fast and those that turn slowly."""
    factor: float
    original: float
    fast: float
    slow: float


@dataclass(frozen=True)
class FosepelRotation:
    dims: int
    base: float
    scaling: Optional[FosepelRamp] = None


@dataclass(frozen=True)
class FosepelAttention:
    """``heads`` query heads over ``kv_heads`` key/value heads, keys of ``dim`` and values of ``vdim``.  ``flavour``:
    "rotary" (q and k normed over all heads, rotated, an element-wise gate), "unit_sink" (biases, q and k normed over all
    heads, a sink of score 0, one gate a head) or "learned_sink" (biases also on the output, a query temperature, capped
    scores, a learned sink a head)."""
    flavour: str
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    rot: Optional[FosepelRotation] = None
    softcap: Optional[float] = None
    q_temp_coef: Optional[float] = None
    q_temp_every: Optional[int] = None


@dataclass(frozen=True)
class FosepelDelta:
    """The delta rule with one decay a head: ``heads`` heads of values of ``vdim`` over ``kv_heads`` heads of q and k of
    ``dim``, short convolutions of ``conv`` taps."""
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int


@dataclass(frozen=True)
class FosepelMemory:
    """The matrix memory: ``heads`` heads with keys of ``dim`` and values of ``vdim``; the gates' logarithms are capped
    at ``gate_cap``."""
    heads: int
    dim: int
    vdim: int
    gate_cap: float


@dataclass(frozen=True)
class FosepelLayer:
    type: str                           # "attention", "parallel" or "parallel_2"
    left: FosepelAttention              # the attention (the only mixer of type "attention")
    right: Any                          # None, FosepelDelta ("parallel") or FosepelMemory ("parallel_2")
    ff: Optional[int]                   # the dense feed-forward's inner size, or None for a layer without one


@dataclass(frozen=True)
class FosepelConfig(ModelConfig):
    vocab: int
    width: int
    layers: Tuple[FosepelLayer, ...]
    norm_eps: float
    logit_softcap: float                # 0: none
    loop_start: int
    loop_stop: int
    loop_times: int                     # 1: no span is repeated

    def run_order(self) -> Tuple[Tuple[int, bool], ...]:
        """(layer, whether the embedding's output is added to the stream before it) in the order in which a token
        passes the layers: the looped span's first layer adds it in every pass but the first."""
        n = len(self.layers)
        out = [(i, False) for i in range(self.loop_start)]
        for rep in range(self.loop_times if self.loop_stop > self.loop_start else 0):
            out += [(i, rep > 0 and i == self.loop_start) for i in range(self.loop_start, self.loop_stop)]
        return tuple(out + [(i, False) for i in range(self.loop_stop, n)])

    # ---- reading -------------------------------------------------------------------
    @classmethod
    def from_dict(cls, data: Dict[str, Any], where: str = "config.json") -> "FosepelConfig":
        r = KeyReader(data, where)
        arch = architecture_name(data, where)
        layers_raw = r.raw("layers")
        if not isinstance(layers_raw, list) or not layers_raw:
            raise ConfigError(f"{where}: key 'layers' must be a list with one entry for each layer")
        layers = tuple(_layer(entry, f"{where}: layers[{i}]") for i, entry in enumerate(layers_raw))
        norm = KeyReader(_obj(r.raw("norm"), f"{where}: norm"), f"{where}: norm")
        loop_raw = r.raw("loop", default=None)
        start, stop, times = 0, 0, 1
        if loop_raw is not None:
            lp = KeyReader(_obj(loop_raw, f"{where}: loop"), f"{where}: loop")
            start, stop = lp.integer("start", minimum=0), lp.integer("stop", minimum=0)
            times = lp.integer("times", default=1, minimum=1)
        cfg = cls(architecture=arch, vocab=r.integer("vocab", minimum=1), width=r.integer("width", minimum=1), layers=layers,
                  norm_eps=norm.number("eps", positive=True), logit_softcap=r.number("logit_softcap", default=0.0) or 0.0,
                  loop_start=start, loop_stop=stop, loop_times=times)
        cfg.validate(where)
        return cfg

    def validate(self, where: str = "config.json") -> None:
        if self.width % 8:
            raise ConfigError(f"{where}: 'width' {self.width} is not supported: the matrix kernels read rows in "
                              f"16-byte pieces, so it must be a multiple of 8")
        if not 0 <= self.loop_start <= self.loop_stop <= len(self.layers):
            raise ConfigError(f"{where}: loop: 'start' {self.loop_start} and 'stop' {self.loop_stop} must lie within the "
                              f"{len(self.layers)} layers, start <= stop")
        for i, layer in enumerate(self.layers):
            at = f"{where}: layers[{i}]"
            a = layer.left
            if a.heads % a.kv_heads:
                raise ConfigError(f"{at}: 'heads' {a.heads} is not a multiple of 'kv_heads' {a.kv_heads}")
            if a.dim > 256 or a.vdim > 1024:
                raise ConfigError(f"{at}: 'dim' above 256 or 'vdim' above 1024 is not supported by the attention kernels")
            if a.rot is not None and (a.rot.dims % 2 or a.rot.dims > a.dim):
                raise ConfigError(f"{at}: 'rot.dims' {a.rot.dims} must be even and at most 'dim' {a.dim}")
            if a.softcap is not None and not a.softcap > 0:
                raise ConfigError(f"{at}: 'softcap' must be positive")
            if a.q_temp_every is not None and a.q_temp_every < 1:
                raise ConfigError(f"{at}: 'q_temp.every' must be at least 1")
            m = layer.right
            if isinstance(m, FosepelDelta):
                if m.heads % m.kv_heads:
                    raise ConfigError(f"{at}: right: 'heads' {m.heads} is not a multiple of 'kv_heads' {m.kv_heads}")
                if not 1 <= m.conv <= 16:
                    raise ConfigError(f"{at}: right: 'conv' {m.conv} taps are not supported (1 to 16)")
            if m is not None and m.dim > 256:
                raise ConfigError(f"{at}: right: 'dim' above 256 is not supported by the scan kernel")
            if isinstance(m, FosepelMemory) and not m.gate_cap > 0:
                raise ConfigError(f"{at}: right: 'gate_cap' must be positive")

    def to_dict(self) -> Dict[str, Any]:
        def attention(a: FosepelAttention):
            out = {"heads": a.heads, "kv_heads": a.kv_heads, "dim": a.dim, "vdim": a.vdim, "scale": a.scale}
            if a.rot is not None:
                out["rot"] = {"dims": a.rot.dims, "base": a.rot.base}
                if a.rot.scaling is not None:
                    s = a.rot.scaling
                    out["rot"]["scaling"] = {"factor": s.factor, "original": s.original, "fast": s.fast, "slow": s.slow}
            if a.softcap is not None:
                out["softcap"] = a.softcap
            if a.q_temp_coef is not None:
                out["q_temp"] = {"coef": a.q_temp_coef, "every": a.q_temp_every}
            return out

        layers = []
        for layer in self.layers:
            if layer.type == "attention":
                mixer = attention(layer.left)
            else:
                m = layer.right
                right = ({"heads": m.heads, "kv_heads": m.kv_heads, "dim": m.dim, "vdim": m.vdim, "conv": m.conv}
                         if isinstance(m, FosepelDelta) else
                         {"heads": m.heads, "dim": m.dim, "vdim": m.vdim, "gate_cap": m.gate_cap})
                mixer = {"left": attention(layer.left), "right": right}
            layers.append({"type": layer.type, "mixer": mixer,
                           "mlp": None if layer.ff is None else {"kind": "dense", "ff": layer.ff}})
        out = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "layers": layers,
               "norm": {"eps": self.norm_eps}}
        if self.logit_softcap:
            out["logit_softcap"] = self.logit_softcap
        if self.loop_times > 1 or self.loop_stop > self.loop_start:
            out["loop"] = {"start": self.loop_start, "stop": self.loop_stop, "times": self.loop_times}
        return out


def _obj(v, where: str) -> Dict[str, Any]:
    if not isinstance(v, dict):
        raise ConfigError(f"{where}: expected an object")
    return v


def _rotation(raw, where: str) -> Optional[FosepelRotation]:
    if raw is None:
        return None
    r = KeyReader(_obj(raw, where), where)
    dims = r.integer("dims", minimum=0)
    if not dims:
        return None
    scaling = None
    sc = r.raw("scaling", default=None)
    if sc is not None:
        s = KeyReader(_obj(sc, where + ".scaling"), where + ".scaling")
        scaling = FosepelRamp(factor=s.number("factor", positive=True), original=s.number("original", positive=True),
                              fast=s.number("fast", positive=True), slow=s.number("slow", positive=True))
    return FosepelRotation(dims=dims, base=r.number("base", positive=True), scaling=scaling)


def _attention(raw, where: str, flavour: str) -> FosepelAttention:
    m = KeyReader(_obj(raw, where), where)
    heads = m.integer("heads", minimum=1)
    dim = m.integer("dim", minimum=1)
    coef = every = None
    qt = m.raw("q_temp", default=None) if flavour == "learned_sink" else None
    if qt is not None:
        t = KeyReader(_obj(qt, where + ".q_temp"), where + ".q_temp")
        coef, every = t.number("coef"), t.integer("every", minimum=1)
    return FosepelAttention(flavour=flavour, heads=heads, kv_heads=m.integer("kv_heads", default=heads, minimum=1), dim=dim,
                            vdim=m.integer("vdim", default=dim, minimum=1), scale=m.number("scale", default=dim ** -0.5),
                            rot=_rotation(m.raw("rot", default=None), where + ".rot") if flavour == "rotary" else None,
                            softcap=m.number("softcap", default=None) if flavour == "learned_sink" else None,
                            q_temp_coef=coef, q_temp_every=every)


def _layer(entry, where: str) -> FosepelLayer:
    r = KeyReader(_obj(entry, where), where)
    kind = r.string("type")
    mw = f"{where}.mixer"
    raw = _obj(r.raw("mixer"), mw)
    if kind == "attention":
        left, right = _attention(raw, mw, "rotary"), None
    elif kind in ("parallel", "parallel_2"):
        pair = KeyReader(raw, mw)
        left = _attention(pair.raw("left"), mw + ".left", "unit_sink" if kind == "parallel" else "learned_sink")
        m = KeyReader(_obj(pair.raw("right"), mw + ".right"), mw + ".right")
        heads, dim = m.integer("heads", minimum=1), m.integer("dim", minimum=1)
        if kind == "parallel":
            right = FosepelDelta(heads=heads, kv_heads=m.integer("kv_heads", default=heads, minimum=1), dim=dim,
                                 vdim=m.integer("vdim", default=dim, minimum=1), conv=m.integer("conv", default=1, minimum=1))
        else:
            right = FosepelMemory(heads=heads, dim=dim, vdim=m.integer("vdim", default=dim, minimum=1),
                                  gate_cap=m.number("gate_cap", positive=True))
    else:
        raise ConfigError(f"{where}: layer type '{kind}' is not known; known are 'attention', 'parallel' and 'parallel_2'")
    mlp_raw = r.raw("mlp", default=None)
    ff = None
    if mlp_raw is not None:
        fw = f"{where}.mlp"
        f = KeyReader(_obj(mlp_raw, fw), fw)
        if f.string("kind", default="dense") != "dense":
            raise ConfigError(f"{fw}: feed-forward kind '{mlp_raw.get('kind')}' is not known; known is 'dense'")
        ff = f.integer("ff", minimum=1)
    return FosepelLayer(type=kind, left=left, right=right, ff=ff)
