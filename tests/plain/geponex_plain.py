"""A plain, slow implementation of the Geponex decoder in float64: one function a mechanism, recurrences as loops over
tokens, attention as a loop over queries.  It shares no code with the package: it reads a configuration as the plain
dictionary of config.json and the weights as a dictionary name -> tensor.

Notation: x is a token's vector in the stream, h what a sublayer reads, W_a the tensor '<layer>.mix.a' (or '.mlp.a'),
stored [out, in] and applied as W h."""
from __future__ import annotations

import json
import math
import os

import torch

F = torch.float64


def read_config(folder: str) -> dict:
    with open(os.path.join(folder, "config.json")) as f:
        return json.load(f)


def read_weights(folder: str, dtype=F):
    from safetensors import safe_open
    out = {}
    with safe_open(os.path.join(folder, "model.safetensors"), framework="pt") as f:
        for name in f.keys():
            out[name] = f.get_tensor(name).to(dtype)
    return out


def sample_greedy(logits):
    return int(torch.argmax(logits))


def rms_norm(v, w, eps):
    """w * v / sqrt(mean(v^2) + eps) over the last dimension."""
    return v / torch.sqrt((v * v).mean(dim=-1, keepdim=True) + eps) * w


def grouped_rms_norm(v, w, eps, groups):
    """The vector in ``groups`` equal consecutive parts, each divided by its own root mean square; then times w."""
    parts = v.reshape(*v.shape[:-1], groups, v.shape[-1] // groups)
    parts = parts / torch.sqrt((parts * parts).mean(dim=-1, keepdim=True) + eps)
    return parts.reshape(v.shape) * w


def token_shift(h, before, mu):
    """h [T, W]: row t becomes h_t + (h_{t-1} - h_t) * mu with the rows as they came in; row 0 takes ``before`` (the
    row of the token in front of this run of tokens, zeros at a sequence's start).  Returns the new rows and the row to
    carry on with."""
    prev = torch.cat([before[None], h[:-1]], dim=0)
    return h + (prev - h) * mu, h[-1].clone()


def rotary_frequencies(dims, base, scaling=None):
    """(f [dims/2], m): f_i = base^(-2i/dims), with ``scaling`` (factor, original, fast, slow) blended towards
    f_i / factor by a ramp over i between two pair indices; m multiplies cos and sin (1 without scaling)."""
    half = dims // 2
    f = [float(base) ** (-2.0 * i / dims) for i in range(half)]
    if scaling is None:
        return torch.tensor(f, dtype=F), 1.0
    factor, original = float(scaling["factor"]), float(scaling["original"])

    def pair_of(turns):
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(pair_of(float(scaling["fast"]))), 0)
    hi = min(math.ceil(pair_of(float(scaling["slow"]))), dims - 1)
    out = []
    for i in range(half):
        ramp = min(1.0, max(0.0, (i - lo) / max(hi - lo, 0.001)))
        out.append(f[i] / factor * ramp + f[i] * (1.0 - ramp))
    return torch.tensor(out, dtype=F), 0.1 * math.log(factor) + 1.0


def rotate_interleaved(v, positions, freq, m):
    """v [T, ..., n]: the first 2 * len(freq) dimensions in pairs (2i, 2i + 1), pair i of the token at position p turned
    by the angle p * freq[i], cos and sin multiplied by m; the other dimensions pass."""
    n = 2 * freq.shape[0]
    ang = positions.to(F)[:, None] * freq[None, :]
    shape = [v.shape[0]] + [1] * (v.dim() - 2) + [freq.shape[0]]
    cos, sin = (torch.cos(ang) * m).reshape(shape), (torch.sin(ang) * m).reshape(shape)
    a, b = v[..., 0:n:2], v[..., 1:n:2]
    out = v.clone()
    out[..., 0:n:2] = a * cos - b * sin
    out[..., 1:n:2] = b * cos + a * sin
    return out


def softmax_attention(q, k, v, q_positions, scale, sink=None):
    """q [T, H, d], k [S, H, d], v [S, H, e], key j at position j: the query at position p sees the keys j <= p.
    Weights exp(s_j) / (sum over the seen keys of exp(s) + exp(sink_h)) (the last term only with ``sink`` [H])."""
    out = torch.zeros(q.shape[0], q.shape[1], v.shape[2], dtype=F)
    for t in range(q.shape[0]):
        n = int(q_positions[t]) + 1
        s = torch.einsum("hd,jhd->hj", q[t], k[:n]) * scale
        mx = s.max(dim=1, keepdim=True).values
        if sink is not None:
            mx = torch.maximum(mx, sink[:, None])
        e = torch.exp(s - mx)
        den = e.sum(dim=1, keepdim=True)
        if sink is not None:
            den = den + torch.exp(sink[:, None] - mx)
        out[t] = torch.einsum("hj,jhe->he", e / den, v[:n])
    return out


class LatentCache:
    """What a latent-attention layer keeps of a sequence: the normed latent and the rotated shared key part of every token."""

    def __init__(self):
        self.c = None
        self.kr = None

    def extend(self, c, kr):
        self.c = c if self.c is None else torch.cat([self.c, c])
        self.kr = kr if self.kr is None else torch.cat([self.kr, kr])


def latent_attention(h, positions, w, m, eps, cache, second):
    """``second``: the variant with a sink in the softmax's denominator and an output gate."""
    H, d, r, e, kv = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    rot = m["rot"]
    freq, mult = rotary_frequencies(rot["dims"], rot["base"], rot.get("scaling"))
    cq = rms_norm(h @ w["dq"].T, w["dq.norm"], eps)
    q = (cq @ w["uq"].T).reshape(-1, H, d + r)
    q_rot = rotate_interleaved(q[..., d:], positions, freq, mult)
    down = h @ w["dkv"].T
    c = rms_norm(down[:, :kv], w["dkv.norm"], eps)
    k_rot = rotate_interleaved(down[:, kv:], positions, freq, mult)
    cache.extend(c, k_rot)
    k_plain = (cache.c @ w["uk"].T).reshape(-1, H, d)
    values = (cache.c @ w["uv"].T).reshape(-1, H, e)
    keys = torch.cat([k_plain, cache.kr[:, None, :].expand(-1, H, -1)], dim=-1)
    queries = torch.cat([q[..., :d], q_rot], dim=-1)
    o = softmax_attention(queries, keys, values, positions, m["scale"], w["sink"] if second else None)
    o = o.reshape(-1, H * e)
    if second:
        o = o * torch.sigmoid(h @ w["g"].T)
    return o @ w["o"].T


def lightning(h, w, m, eps, state):
    """state [H, d, e] is carried from token to token; returns the output and leaves the state as after the last token."""
    H, d, e = m["heads"], m["dim"], m["vdim"]
    silu = torch.nn.functional.silu
    q = silu(h @ w["q"].T).reshape(-1, H, d)
    k = silu(h @ w["k"].T).reshape(-1, H, d)
    v = silu(h @ w["v"].T).reshape(-1, H, e)
    decay = torch.tensor(m["decay"], dtype=F)
    o = torch.zeros(h.shape[0], H, e, dtype=F)
    for t in range(h.shape[0]):
        state.mul_(decay[:, None, None]).add_(torch.einsum("hd,he->hde", k[t], v[t]))
        o[t] = torch.einsum("hde,hd->he", state, q[t])
    o = rms_norm(o.reshape(-1, H * e), w["norm"], eps) * torch.sigmoid(h @ w["g"].T)
    return o @ w["o"].T


def xielu(z, p, q):
    sp = torch.nn.functional.softplus
    pos = sp(p) * z * z + z / 2
    neg = (0.5 + sp(q)) * (torch.exp(torch.clamp(z, max=0.0)) - 1.0 - z) + z / 2
    return torch.where(z > 0, pos, neg)


def dense_ff(h, w):
    z = h @ w["up"].T + w["up.b"]
    return xielu(z, w["act"][0], w["act"][1]) @ w["down"].T + w["down.b"]


def expert(h, gate, up, down, limit):
    g = torch.clamp(h @ gate.T, max=limit)
    u = torch.clamp(h @ up.T, min=-limit, max=limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ down.T


def route(h, router, top, scale, margins=None):
    """(ids [T, top], weights [T, top]): the experts with the largest sigmoid scores, the scores over their sum, scaled.
    ``margins`` gets, for every token, how far the last chosen logit lies above the first that is not, as a part of the
    largest logit's size."""
    z = h @ router.T
    s = torch.sigmoid(z)
    if margins is not None and top < z.shape[1]:
        ranked = torch.sort(z, dim=1, descending=True).values
        margins.append((ranked[:, top - 1] - ranked[:, top]) / z.abs().max(dim=1).values.clamp_min(1e-9))
    chosen = torch.topk(s, top, dim=-1)
    return chosen.indices, chosen.values / (chosen.values.sum(dim=-1, keepdim=True) + 1e-20) * scale


def moe_ff(h, w, f, margins=None):
    ids, weights = route(h, w["router"], f["router"]["top"], f["router"]["scale"], margins)
    out = torch.zeros(h.shape[0], w["e0.down"].shape[0], dtype=F)
    for t in range(h.shape[0]):
        for e, wt in zip(ids[t].tolist(), weights[t]):
            out[t] += wt * expert(h[t:t + 1], w[f"e{e}.gate"], w[f"e{e}.up"], w[f"e{e}.down"], f["expert"]["limit"])[0]
    if f.get("shared") is not None:
        out = out + expert(h, w["shared.gate"], w["shared.up"], w["shared.down"], f["shared"]["limit"])
    return out


def owner_of(layers, i):
    while "weights_of" in layers[i] and layers[i]["weights_of"] is not None:
        i = layers[i]["weights_of"]
    return i


def sub(weights, prefix):
    return {k[len(prefix):]: v.to(F) for k, v in weights.items() if k.startswith(prefix)}


class Sequence:
    """What every layer keeps of one sequence, and how many tokens it has seen."""

    def __init__(self, config):
        self.length = 0
        self.layers = []
        for layer in config["layers"]:
            m = layer["mixer"]
            mix = (torch.zeros(m["heads"], m["dim"], m["vdim"], dtype=F) if layer["type"] == "lightning" else LatentCache())
            self.layers.append({"before": torch.zeros(config["width"], dtype=F), "mix": mix})


def forward(config, weights, tokens, seq=None, trace=None, margins=None):
    """Runs ``tokens`` after what ``seq`` has seen; returns logits [T, vocab].  ``trace``: a list that takes the stream
    after every layer.  ``margins``: a list that takes every router's margins (see ``route``)."""
    seq = seq if seq is not None else Sequence(config)
    eps, groups, alpha = config["norm"]["eps"], config["norm"]["groups"], config["postln_alpha"]
    positions = torch.arange(seq.length, seq.length + len(tokens))
    x = weights["embed"].to(F)[torch.as_tensor(tokens, dtype=torch.long)]
    for i, layer in enumerate(config["layers"]):
        p = f"l{owner_of(config['layers'], i)}."
        kept = seq.layers[i]
        h, kept["before"] = token_shift(x, kept["before"], weights[p + "shift"].to(F))
        w = sub(weights, p + "mix.")
        if layer["type"] == "lightning":
            y = lightning(h, w, layer["mixer"], eps, kept["mix"])
        else:
            y = latent_attention(h, positions, w, layer["mixer"], eps, kept["mix"], layer["type"] == "latent_attention_2")
        x = grouped_rms_norm(alpha * x + y, weights[p + "norm1"].to(F), eps, groups)
        f = layer.get("mlp")
        if f is not None:
            w = sub(weights, p + "mlp.")
            y = dense_ff(x, w) if f["kind"] == "dense" else moe_ff(x, w, f, margins)
            x = grouped_rms_norm(alpha * x + y, weights[p + "norm2"].to(F), eps, groups)
        if trace is not None:
            trace.append(x.clone())
    seq.length += len(tokens)
    x = grouped_rms_norm(x, weights["final.norm"].to(F), eps, groups)
    return x @ weights["embed"].to(F).T
