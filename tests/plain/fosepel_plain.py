"""Plain, slow implementation of the Fosepel decoder: the oracle of its tests.

Whole sequences, no cache, no batching, one function for each mechanism, every recurrence a loop
over the tokens.  It shares no code with the package: config.json is read with ``json``, the
weights with the ``safetensors`` library, and everything is computed with torch on the CPU in
``float64`` (or ``float32``).

Notation.  T tokens at positions 0..T-1, x the residual stream [T, width], h a mixer's input (the
normed stream).  W[name] is stored [out, in] and applied as W h.  rms(y) = y / sqrt(mean(y^2) + eps).

* layer:        x <- x + N_1b(mixer(N_1(x)));  x <- x + N_2b(ff(N_2(x)));  N(y) = rms(y) * w.
* loop:         layers start..stop-1 run ``times`` times; before every pass but the first the embedding's
                output is added to x.
* attention:    q and k normed over all heads together (weights), rotated on the first ``dims`` dimensions of a head
                (pairs (i, i + dims/2), frequencies blended by a ramp, cos and sin scaled), ordinary causal softmax,
                result times sigmoid(G h) element by element.
* parallel:     half of rms(left) * w_l + rms(right) * w_r, where left is a softmax attention (biases, q and k normed
                over all heads, a sink of score 0 in the denominator, one gate a head) and right the gated delta rule
                (short convolutions with silu, unit q and k, S <- g S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q).
* parallel_2:   the same sum of a softmax attention (biases, a query temperature that grows with the position, capped
                scores, a learned sink a head) and the matrix memory with exponential gates (a running maximum m keeps the
                exponentials bounded).
"""
from __future__ import annotations

import json
import math
import os
from typing import Dict, List, Optional, Sequence

import torch


def read_config(folder: str) -> dict:
    with open(os.path.join(folder, "config.json")) as f:
        return json.load(f)


def read_weights(folder: str, dtype=torch.float64) -> Dict[str, torch.Tensor]:
    from safetensors import safe_open
    out = {}
    with safe_open(os.path.join(folder, "model.safetensors"), framework="pt") as f:
        for name in f.keys():
            out[name] = f.get_tensor(name).to(dtype)
    return out


# --------------------------------------------------------------------------- small pieces


def rms(y: torch.Tensor, eps: float) -> torch.Tensor:
    return y / torch.sqrt((y * y).mean(dim=-1, keepdim=True) + eps)


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


def softplus(z: torch.Tensor) -> torch.Tensor:
    return torch.where(z > 30.0, z, torch.log1p(torch.exp(torch.clamp(z, max=30.0))))


def log_sigmoid(z: torch.Tensor) -> torch.Tensor:
    return -softplus(-z)


def ramped_frequencies(rot: dict):
    """(f [dims/2], m): f_i = base^(-2i/dims).  With ``scaling`` (factor, original, fast, slow): let
    n(t) = dims ln(original / (2 pi t)) / (2 ln base), lo = max(floor(n(fast)), 0), hi = min(ceil(n(slow)), dims - 1) and
    r_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1); then f_i <- f_i / factor * r_i + f_i (1 - r_i) and cos and sin are
    multiplied by m = 0.1 ln(factor) + 1."""
    dims, base = int(rot["dims"]), float(rot["base"])
    f = [base ** (-2.0 * i / dims) for i in range(dims // 2)]
    m = 1.0
    sc = rot.get("scaling")
    if sc:
        factor, orig = float(sc["factor"]), float(sc["original"])

        def n(turns):
            return dims * math.log(orig / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

        lo = max(math.floor(n(float(sc["fast"]))), 0)
        hi = min(math.ceil(n(float(sc["slow"]))), dims - 1)
        for i in range(len(f)):
            r = min(1.0, max(0.0, (i - lo) / max(hi - lo, 0.001)))
            f[i] = f[i] / factor * r + f[i] * (1.0 - r)
        m = 0.1 * math.log(factor) + 1.0
    return f, m


def rotate(x: torch.Tensor, rot: Optional[dict]) -> torch.Tensor:
    """x [T, heads, dim]: the first ``dims`` dimensions of every head turn in pairs (i, i + dims/2) by position * f_i."""
    if not rot or not int(rot.get("dims", 0)):
        return x
    dims = int(rot["dims"])
    half = dims // 2
    f, m = ramped_frequencies(rot)
    pos = torch.arange(x.shape[0], dtype=x.dtype)
    angle = pos[:, None] * torch.tensor(f, dtype=x.dtype)[None, :]            # [T, half]
    c, s = (torch.cos(angle) * m)[:, None, :], (torch.sin(angle) * m)[:, None, :]
    a, b = x[..., :half], x[..., half:dims]
    return torch.cat([a * c - b * s, b * c + a * s, x[..., dims:]], dim=-1)


def causal_softmax_attention(q, k, v, scale: float, cap: Optional[float] = None, sink: Optional[torch.Tensor] = None):
    """q [T, H, d], k [T, G, d], v [T, G, e] -> [T, H, e].  Head h reads key/value head h // (H / G); position t sees
    j <= t; score = q . k * scale, then cap * tanh(score / cap) where a cap is given; p_j = exp(s_j) / (sum exp(s) + exp(sink_h))
    where ``sink`` [H] is given (a term without key or value)."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros((T, H, v.shape[-1]), dtype=q.dtype)
    for h in range(H):
        g = h // (H // G)
        for t in range(T):
            s = (k[:t + 1, g] @ q[t, h]) * scale
            if cap:
                s = cap * torch.tanh(s / cap)
            top = s.max() if sink is None else torch.maximum(s.max(), sink[h])
            e = torch.exp(s - top)
            den = e.sum() + (0.0 if sink is None else torch.exp(sink[h] - top))
            out[t, h] = (e / den) @ v[:t + 1, g]
    return out


def short_convolution(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """x [T, C], w [C, taps]: y_t[c] = sum_j w[c, j] x_(t - taps + 1 + j)[c], zeros before the first token."""
    T, C = x.shape
    taps = w.shape[1]
    padded = torch.cat([torch.zeros((taps - 1, C), dtype=x.dtype), x], dim=0)
    y = torch.zeros_like(x)
    for j in range(taps):
        y = y + padded[j:j + T] * w[:, j][None, :]
    return y


def gated_delta_rule(q, k, v, beta, g):
    """q, k [T, G, d], v [T, H, e], beta and g [T, H] -> [T, H, e].  For each head, with S [d, e] zero at the start:
    S <- g_t S; u = beta_t (v_t - S^T k_t); S <- S + k_t u^T; o_t = S^T q_t."""
    T, H, e = v.shape
    G, d = k.shape[1], k.shape[2]
    out = torch.zeros_like(v)
    for h in range(H):
        kh = h // (H // G)
        S = torch.zeros((d, e), dtype=v.dtype)
        for t in range(T):
            S = g[t, h] * S
            u = beta[t, h] * (v[t, h] - S.t() @ k[t, kh])
            S = S + torch.outer(k[t, kh], u)
            out[t, h] = S.t() @ q[t, kh]
    return out


def matrix_memory(q, k, v, i_gate, f_gate):
    """q, k [T, H, d], v [T, H, e], i_gate and f_gate [T, H] (logarithms of the input and forget gates) -> [T, H, e].
    For each head, with S [d, e], n [d] and m zero at the start: m_t = max(f + m, i); S <- exp(f + m - m_t) S +
    exp(i - m_t) k v^T; n likewise with k alone; o_t = S^T q / (max(|n . q|, exp(-m_t)) + 1e-6)."""
    T, H, e = v.shape
    d = k.shape[2]
    out = torch.zeros_like(v)
    for h in range(H):
        S = torch.zeros((d, e), dtype=v.dtype)
        n = torch.zeros(d, dtype=v.dtype)
        m = torch.zeros((), dtype=v.dtype)
        for t in range(T):
            m_new = torch.maximum(f_gate[t, h] + m, i_gate[t, h])
            a, b = torch.exp(f_gate[t, h] + m - m_new), torch.exp(i_gate[t, h] - m_new)
            S = a * S + b * torch.outer(k[t, h], v[t, h])
            n = a * n + b * k[t, h]
            m = m_new
            den = torch.maximum((n @ q[t, h]).abs(), torch.exp(-m)) + 1e-6
            out[t, h] = (S.t() @ q[t, h]) / den
    return out


# --------------------------------------------------------------------------- mixers


def _lin(W, name, h, bias: bool = False):
    y = h @ W[name].t()
    return y + W[name + ".b"] if bias else y


def attention_mixer(m: dict, W, p: str, h, eps: float):
    T = h.shape[0]
    H, G, d = int(m["heads"]), int(m["kv_heads"]), int(m["dim"])
    e = int(m.get("vdim", d))
    q = rms(_lin(W, p + "q", h), eps) * W[p + "q.norm"]
    k = rms(_lin(W, p + "k", h), eps) * W[p + "k.norm"]
    v = _lin(W, p + "v", h)
    q, k = rotate(q.view(T, H, d), m.get("rot")), rotate(k.view(T, G, d), m.get("rot"))
    o = causal_softmax_attention(q, k, v.view(T, G, e), float(m["scale"]))
    o = o.reshape(T, H * e) * torch.sigmoid(_lin(W, p + "g", h))
    return _lin(W, p + "o", o)


def left_with_unit_sink(m: dict, W, p: str, h, eps: float):
    """The softmax attention beside the gated delta rule: biases, q and k normed over all heads, no rotation, a sink of
    score 0, one gate a head."""
    T = h.shape[0]
    H, G, d = int(m["heads"]), int(m["kv_heads"]), int(m["dim"])
    e = int(m.get("vdim", d))
    q = rms(_lin(W, p + "q", h, True), eps) * W[p + "q.norm"]
    k = rms(_lin(W, p + "k", h, True), eps) * W[p + "k.norm"]
    v = _lin(W, p + "v", h, True)
    o = causal_softmax_attention(q.view(T, H, d), k.view(T, G, d), v.view(T, G, e), float(m["scale"]),
                                 sink=torch.zeros(H, dtype=h.dtype))
    o = o * torch.sigmoid(_lin(W, p + "g", h))[:, :, None]
    return _lin(W, p + "o", o.reshape(T, H * e))


def left_with_learned_sink(m: dict, W, p: str, h):
    """The softmax attention beside the matrix memory: biases (also on the output), a query temperature by position, capped
    scores, a learned sink a head."""
    T = h.shape[0]
    H, G, d = int(m["heads"]), int(m["kv_heads"]), int(m["dim"])
    e = int(m.get("vdim", d))
    q = _lin(W, p + "q", h, True).view(T, H, d)
    k = _lin(W, p + "k", h, True).view(T, G, d)
    v = _lin(W, p + "v", h, True).view(T, G, e)
    qt = m.get("q_temp")
    if qt:
        pos = torch.arange(T, dtype=h.dtype)
        q = q * (1.0 + float(qt["coef"]) * torch.log(torch.floor((pos + 1.0) / float(qt["every"])) + 1.0))[:, None, None]
    cap = m.get("softcap")
    o = causal_softmax_attention(q, k, v, float(m["scale"]), cap=float(cap) if cap else None, sink=W[p + "sink"])
    return _lin(W, p + "o", o.reshape(T, H * e), True)


def right_gated_delta(m: dict, W, p: str, h, eps: float):
    T = h.shape[0]
    H, G, d, e = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    q = silu(short_convolution(_lin(W, p + "q", h), W[p + "q.conv"])).view(T, G, d)
    k = silu(short_convolution(_lin(W, p + "k", h), W[p + "k.conv"])).view(T, G, d)
    v = silu(short_convolution(_lin(W, p + "v", h), W[p + "v.conv"])).view(T, H, e)
    q = q / torch.sqrt((q * q).sum(dim=-1, keepdim=True) + 1e-6) * d ** -0.5
    k = k / torch.sqrt((k * k).sum(dim=-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(_lin(W, p + "b", h))
    g = torch.exp(-torch.exp(W[p + "A_log"]) * softplus(_lin(W, p + "a", h) + W[p + "dt_bias"]))
    o = gated_delta_rule(q, k, v, beta, g)
    o = rms(o, eps) * W[p + "norm"] * silu(_lin(W, p + "g", h)).view(T, H, e)
    return _lin(W, p + "o", o.reshape(T, H * e))


def right_matrix_memory(m: dict, W, p: str, h, eps: float):
    T = h.shape[0]
    H, d, e = int(m["heads"]), int(m["dim"]), int(m["vdim"])
    cap = float(m["gate_cap"])
    q = _lin(W, p + "q", h).view(T, H, d) * d ** -0.5
    k = _lin(W, p + "k", h).view(T, H, d)
    v = _lin(W, p + "v", h).view(T, H, e)
    i_gate = cap * torch.tanh(_lin(W, p + "i", h, True) / cap)
    f_gate = log_sigmoid(cap * torch.tanh(_lin(W, p + "f", h, True) / cap))
    o = matrix_memory(q, k, v, i_gate, f_gate)
    o = rms(o, eps).reshape(T, H * e) * W[p + "norm"] * torch.sigmoid(_lin(W, p + "g", h))
    return _lin(W, p + "o", o)


def mixer(layer: dict, W, p: str, h, eps: float):
    kind, m = layer["type"], layer["mixer"]
    if kind == "attention":
        return attention_mixer(m, W, p, h, eps)
    if kind == "parallel":
        left = left_with_unit_sink(m["left"], W, p + "left.", h, eps)
        right = right_gated_delta(m["right"], W, p + "right.", h, eps)
    elif kind == "parallel_2":
        left = left_with_learned_sink(m["left"], W, p + "left.", h)
        right = right_matrix_memory(m["right"], W, p + "right.", h, eps)
    else:
        raise ValueError(kind)
    return 0.5 * (rms(left, eps) * W[p + "left.out"] + rms(right, eps) * W[p + "right.out"])


def feed_forward(W, p: str, h):
    return _lin(W, p + "down", silu(_lin(W, p + "gate", h)) * _lin(W, p + "up", h))


# --------------------------------------------------------------------------- the model


def run_order(cfg: dict) -> List[int]:
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return list(range(n))
    a, b, times = int(loop["start"]), int(loop["stop"]), int(loop.get("times", 1))
    return list(range(a)) + list(range(a, b)) * times + list(range(b, n))


def forward(cfg: dict, W: Dict[str, torch.Tensor], tokens: Sequence[int], layers_out: Optional[list] = None) -> torch.Tensor:
    """Logits [T, vocab] of the whole sequence.  ``layers_out``: a list that receives x after every layer run."""
    eps = float(cfg["norm"]["eps"])
    x = W["embed"][torch.tensor(list(tokens), dtype=torch.long)]
    first = x.clone()
    loop = cfg.get("loop")
    start = int(loop["start"]) if loop else -1
    seen_start = 0
    for i in run_order(cfg):
        if loop and i == start and int(loop["stop"]) > start:
            if seen_start:
                x = x + first
            seen_start += 1
        layer, p = cfg["layers"][i], f"l{i}."
        h = rms(x, eps) * W[p + "norm1"]
        x = x + rms(mixer(layer, W, p + "mix.", h, eps), eps) * W[p + "norm1b"]
        if layer.get("mlp"):
            h = rms(x, eps) * W[p + "norm2"]
            x = x + rms(feed_forward(W, p + "mlp.", h), eps) * W[p + "norm2b"]
        if layers_out is not None:
            layers_out.append(x.clone())
    y = rms(x, eps) * W["final.norm"]
    logits = y @ W["embed"].t()
    cap = cfg.get("logit_softcap")
    return float(cap) * torch.tanh(logits / float(cap)) if cap else logits


def sample_greedy(logits_row: torch.Tensor) -> int:
    return int(torch.argmax(logits_row))
