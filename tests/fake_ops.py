"""A stand-in for the CUDA extension, in torch on the CPU, for tests of the host-side logic
(cache manager, batching, run order, scheduler) on a machine without a GPU.

It has the functions of the extension module with the same arguments and the same
in-place effects.  It is test equipment: the package never selects it; a test installs it
with ``vt_transformer_b200.ops.use_backend``.  Kernels themselves are tested on the GPU
against the plain implementation, not against this file.
"""
from __future__ import annotations

import torch


def embedding(table, ids, out, status=None, scale=1.0):
    idx = ids.long()
    ok = (idx >= 0) & (idx < table.shape[0])
    out.zero_()
    out[ok] = table[idx[ok]].float() * scale
    if status is not None and bool((idx >= table.shape[0]).any()):
        status[0] = 1


def logits_scale_cap(logits, scale, cap):
    logits.mul_(scale)
    if cap > 0:
        logits.copy_(cap * torch.tanh(logits / cap))


def _normed_first(d, post_weight, post_eps, post_mult):
    """A delta that is normed and scaled before it is added."""
    if post_weight is None:
        return d
    return post_mult * post_weight * d * torch.rsqrt((d * d).mean(dim=-1, keepdim=True) + post_eps)


def rmsnorm(x, delta, weight, eps, out, rows=None, status=None, post_weight=None, post_eps=0.0, post_mult=1.0, groups=1,
            x_scale=1.0, write_normed=False):
    idx = torch.arange(x.shape[0]) if rows is None else rows.long()
    v = x[idx] * x_scale
    if delta is not None:
        if delta.dim() == 3:                     # the unadded shares of a product
            delta = delta.sum(dim=0)
        v = v + _normed_first(delta[idx].float(), post_weight, post_eps, post_mult)
    if delta is not None or x_scale != 1.0:
        x[idx] = v
    parts = v.view(v.shape[0], groups, -1)
    y = weight * (parts * torch.rsqrt((parts * parts).mean(dim=-1, keepdim=True) + eps)).reshape(v.shape)
    if out is not None:
        out.copy_(y.to(out.dtype))
    if write_normed:
        x[idx] = y


def silu_mul(gu, out, interleave=0):
    inter = out.shape[1]
    if interleave:
        pairs = gu.view(gu.shape[0], inter // 8, 2, 8).float()
        g, u = pairs[:, :, 0].reshape(-1, inter), pairs[:, :, 1].reshape(-1, inter)
    else:
        g, u = gu[:, :inter].float(), gu[:, inter:].float()
    out.copy_((g / (1.0 + torch.exp(-g)) * u).to(out.dtype))


def _rotate(x, cs):
    half = x.shape[-1] // 2
    a, b = x[..., :half].float(), x[..., half:].float()
    c, s = cs[:, None, :, 0], cs[:, None, :, 1]
    return torch.cat([a * c - b * s, b * c + a * s], dim=-1)


def rope_store(qkv, positions, cos_sin, k_cache, v_cache, token_seq, block_table, heads, kv_heads, head_dim,
               store, status=None):
    T = qkv.shape[0]
    live = token_seq >= 0
    qd, kd = heads * head_dim, kv_heads * head_dim
    page_size = k_cache.shape[2]
    q = qkv[:, :qd].view(T, heads, head_dim)
    k = qkv[:, qd:qd + kd].view(T, kv_heads, head_dim)
    v = qkv[:, qd + kd:].view(T, kv_heads, head_dim)
    pos = positions.long().clamp(min=0)
    if cos_sin is not None:
        cs = cos_sin[pos]
        q_rot = _rotate(q, cs).to(qkv.dtype)
        k_rot = _rotate(k, cs).to(qkv.dtype)
        q[live] = q_rot[live]
    else:
        k_rot = k
    if not store:
        return
    for t in range(T):
        if not bool(live[t]):
            continue
        p = int(positions[t])
        page = int(block_table[int(token_seq[t]), p // page_size])
        assert 0 <= page < k_cache.shape[0], "bad page"
        k_cache[page, :, p % page_size, :] = k_rot[t]
        v_cache[page, :, p % page_size, :] = v[t]


def gemm_simt(a, w, bias, c):
    y = a.float() @ w.float().t()
    if bias is not None:
        y = y + bias
    c.copy_(y.to(c.dtype))


def attention_simt(qkv, out, k_cache, v_cache, positions, token_seq, block_table, heads, kv_heads, head_dim,
                   window, scale, status=None):
    T = qkv.shape[0]
    page_size = k_cache.shape[2]
    g = heads // kv_heads
    q = qkv[:, :heads * head_dim].view(T, heads, head_dim).float()
    for t in range(T):
        s = int(token_seq[t])
        if s < 0:
            out[t] = 0
            continue
        p = int(positions[t])
        first = max(0, p - window + 1) if window > 0 else 0
        js = torch.arange(first, p + 1)
        pages = block_table[s, (js // page_size)].long()
        assert bool((pages >= 0).all()), "attention reads a page that is not held"
        keys = k_cache[pages, :, js % page_size, :].float()      # [J, kv_heads, d]
        vals = v_cache[pages, :, js % page_size, :].float()
        for h in range(heads):
            sc = (keys[:, h // g, :] @ q[t, h]) * scale
            pr = torch.softmax(sc, dim=0)
            out[t, h * head_dim:(h + 1) * head_dim] = (pr @ vals[:, h // g, :]).to(out.dtype)


def argmax(logits, out):
    out.copy_(torch.argmax(logits, dim=-1).to(torch.int32))


def sample(logits, temperature, top_k, top_p, u, out):
    for r in range(logits.shape[0]):
        t = float(temperature[r])
        k = int(top_k[r])
        if not t > 0 or k == 1:
            out[r] = int(torch.argmax(logits[r]))
            continue
        z = logits[r].double() / t
        keep = torch.ones_like(z, dtype=torch.bool)
        if 0 < k < z.numel():
            keep &= z >= torch.topk(z, k).values[-1]
        e = torch.where(keep, torch.exp(z - z.max()), torch.zeros_like(z))
        p = float(top_p[r])
        if p < 1.0:
            order = torch.argsort(e, descending=True)
            c = torch.cumsum(e[order], 0)
            n = int(torch.searchsorted(c, torch.tensor(p * float(c[-1]), dtype=torch.float64))) + 1
            thr = e[order[min(n, z.numel()) - 1]]
            e = torch.where(e >= thr, e, torch.zeros_like(e))
        c = torch.cumsum(e, 0)
        idx = int(torch.searchsorted(c, torch.tensor(float(u[r]) * float(c[-1]), dtype=torch.float64), right=True))
        out[r] = min(idx, z.numel() - 1)


# ---- the kernels of the layer norm, the general attention, the recurrent mixers and the PolyNorm activation ----


def layernorm(x, delta, weight, eps, out, rows=None, status=None, post_weight=None, post_eps=0.0, post_mult=1.0):
    idx = torch.arange(x.shape[0]) if rows is None else rows.long()
    v = x[idx]
    if delta is not None:
        v = v + _normed_first(delta[idx].float(), post_weight, post_eps, post_mult)
        x[idx] = v
    dev = v - v.mean(dim=-1, keepdim=True)
    out.copy_((weight * dev * torch.rsqrt((dev * dev).mean(dim=-1, keepdim=True) + eps)).to(out.dtype))


def polynorm(z, coefficients, eps, out, n_mean=0):
    a, b, c, e = [float(v) for v in coefficients]
    zf = z.float()
    count = n_mean if n_mean > 0 else z.shape[1]
    n = lambda y: y * torch.rsqrt((y * y).sum(dim=-1, keepdim=True) / count + eps)
    out.copy_((a * n(zf) + b * n(zf * zf) + c * n(zf * zf * zf) + e).to(out.dtype))


def head_norm_gate(o, y, gate_col, weight, weight_per_channel, eps, act, out, out_col, out_scale, heads, v_dim, token_seq=None):
    T = o.shape[0]
    oh = o.view(T, heads, v_dim)
    n = oh * torch.rsqrt((oh * oh).mean(dim=-1, keepdim=True) + eps)
    w = weight.view(heads, v_dim) if weight_per_channel else weight.view(1, v_dim)
    g = y[:, gate_col:gate_col + heads * v_dim].float().view(T, heads, v_dim)
    g = g * torch.sigmoid(g) if act == 0 else torch.sigmoid(g)
    out[:, out_col:out_col + heads * v_dim] = (out_scale * n * w * g).reshape(T, heads * v_dim).to(out.dtype)
    if token_seq is not None:
        out[token_seq < 0, out_col:out_col + heads * v_dim] = 0


def _sequences(cu_q, rows):
    cu = cu_q.tolist()
    return [(int(rows[i]), cu[i], cu[i + 1]) for i in range(len(cu) - 1) if cu[i + 1] > cu[i]]


def gla_scan(y, q_col, k_col, v_col, a_col, a2, a2_bias, inv_tau, q_scale, state, cu_q, rows, o, heads, dim, v_dim, status=None,
             most_threads=0):
    rank = a2.shape[1]
    yf = y.float()
    z = yf[:, a_col:a_col + rank] @ a2.t() + a2_bias
    alpha = torch.exp(torch.nn.functional.logsigmoid(z) * inv_tau).view(-1, heads, dim)
    q = yf[:, q_col:q_col + heads * dim].view(-1, heads, dim) * q_scale
    k = yf[:, k_col:k_col + heads * dim].view(-1, heads, dim)
    v = yf[:, v_col:v_col + heads * v_dim].view(-1, heads, v_dim)
    for row, a, b in _sequences(cu_q, rows):
        S = state[row].clone()
        for t in range(a, b):
            S = alpha[t][:, :, None] * S + k[t][:, :, None] * v[t][:, None, :]
            o[t] = torch.einsum("hdv,hd->hv", S, q[t]).reshape(-1)
        state[row] = S


def delta_scan(y, r_col, k_col, v_col, a_col, w1_col, w2, w0, a_bias, decay_rate, key_eps, state, cu_q, rows, o, heads, dim,
               status=None, most_threads=0):
    rank = w2.shape[1]
    yf = y.float()
    n = heads * dim
    w = torch.exp(-decay_rate * torch.sigmoid(torch.tanh(yf[:, w1_col:w1_col + rank]) @ w2.t() + w0)).view(-1, heads, dim)
    a = torch.sigmoid(yf[:, a_col:a_col + n] + a_bias).view(-1, heads, dim)
    r = yf[:, r_col:r_col + n].view(-1, heads, dim)
    k = yf[:, k_col:k_col + n].view(-1, heads, dim)
    v = yf[:, v_col:v_col + n].view(-1, heads, dim)
    u = k / torch.sqrt((k * k).sum(dim=-1, keepdim=True) + key_eps)
    for row, lo, hi in _sequences(cu_q, rows):
        S = state[row].clone()
        for t in range(lo, hi):
            uS = torch.einsum("hd,hdv->hv", u[t], S)
            S = w[t][:, :, None] * S - (a[t] * u[t])[:, :, None] * uS[:, None, :] + k[t][:, :, None] * v[t][:, None, :]
            o[t] = torch.einsum("hdv,hd->hv", S, r[t]).reshape(-1)
        state[row] = S


def attention_prepare(y, q_col, k_col, v_col, positions, token_seq, frequencies, norm_eps, k_cache, v_cache, block_table,
                      heads, kv_heads, dim, v_dim, store, status=None, v_heads=None, q_weight=None, k_weight=None, norm_first=False,
                      whole_projection=False, rot_mult=1.0, q_temp_coef=0.0, q_temp_every=1):
    T = y.shape[0]
    page_size = k_cache.shape[2]
    live = token_seq >= 0
    v_heads = kv_heads if v_heads is None else v_heads

    def normed(x, w):
        if norm_eps >= 0 and whole_projection:       # one mean square over all heads, a weight for every channel
            flat = x.reshape(x.shape[0], -1)
            flat = flat * torch.rsqrt((flat * flat).mean(dim=-1, keepdim=True) + norm_eps)
            return (flat * w if w is not None else flat).reshape(x.shape)
        if norm_eps >= 0:
            x = x * torch.rsqrt((x * x).mean(dim=-1, keepdim=True) + norm_eps)
            if w is not None:
                x = x * w
        return x

    def turn(x, w=None):                           # x [T, n, dim] float
        if norm_first:
            x = normed(x, w)
        if frequencies is not None and frequencies.numel():
            half = frequencies.numel()
            ang = positions.float()[:, None] * frequencies.float()[None, :]
            c, s = torch.cos(ang)[:, None, :] * rot_mult, torch.sin(ang)[:, None, :] * rot_mult
            a, b = x[..., :half].clone(), x[..., half:2 * half].clone()
            x[..., :half] = a * c - b * s
            x[..., half:2 * half] = b * c + a * s
        if not norm_first:
            x = normed(x, w)
        return x

    q = turn(y[:, q_col:q_col + heads * dim].float().view(T, heads, dim).clone(), q_weight)
    if q_temp_coef != 0.0:
        steps = torch.div(positions.clamp(min=0) + 1, q_temp_every, rounding_mode="floor").float()
        q = q * (1.0 + q_temp_coef * torch.log(steps + 1.0))[:, None, None]
    y[:, q_col:q_col + heads * dim] = q.reshape(T, heads * dim).to(y.dtype)
    if not store:
        return
    k = turn(y[:, k_col:k_col + kv_heads * dim].float().view(T, kv_heads, dim).clone(), k_weight)
    v = y[:, v_col:v_col + v_heads * v_dim].view(T, v_heads, v_dim)
    for t in range(T):
        if not bool(live[t]):
            continue
        p = int(positions[t])
        page = int(block_table[int(token_seq[t]), p // page_size])
        assert page >= 0, "a key is stored into a page that is not held"
        k_cache[page, :, p % page_size, :] = k[t].to(k_cache.dtype)
        v_cache[page, :, p % page_size, :] = v[t].to(v_cache.dtype)


def attention_general(y, q_col, out, out_col, out_scale, k_cache, v_cache, positions, token_seq, block_table, heads, kv_heads,
                      dim, v_dim, window, chunk, scale, status=None, keep_first=0, maps=1, lam=0.0, sub_eps=0.0, sinks=None,
                      values_in_keys=False, softcap=0.0, gate_mode=0, gate_col=0):
    T = y.shape[0]
    page_size = k_cache.shape[2]
    g = heads // kv_heads
    q = y[:, q_col:q_col + heads * maps * dim].float().view(T, heads * maps, dim)
    for t in range(T):
        s = int(token_seq[t])
        if s < 0:
            out[t, out_col:out_col + heads * v_dim] = 0
            continue
        p = int(positions[t])
        first = max(0, p - window + 1) if window > 0 else 0
        if chunk > 0:
            first = max(first, (p // chunk) * chunk)
        js = torch.cat([torch.arange(0, min(keep_first, first)), torch.arange(first, p + 1)])
        pages = block_table[s, (js // page_size)].long()
        assert bool((pages >= 0).all()), "attention reads a page that is not held"
        keys = k_cache[pages, :, js % page_size, :].float()
        vals = keys[..., :v_dim] if values_in_keys else v_cache[pages, :, js % page_size, :].float()
        for h in range(heads):
            if maps == 1:
                sc = (keys[:, h // g, :] @ q[t, h]) * scale
                if softcap > 0:
                    sc = softcap * torch.tanh(sc / softcap)
                if sinks is not None:            # one more term in the denominator, without a value
                    pr = torch.softmax(torch.cat([sc, sinks[h:h + 1].float()]), dim=0)[:-1]
                else:
                    pr = torch.softmax(sc, dim=0)
                o = out_scale * (pr @ vals[:, h // g, :])
                if gate_mode == 1:
                    o = o * torch.sigmoid(y[t, gate_col + h].float())
                elif gate_mode == 2:
                    o = o * torch.sigmoid(y[t, gate_col + h * v_dim:gate_col + (h + 1) * v_dim].float())
            else:
                a = [torch.softmax((keys[:, (h // g) * 2 + m, :] @ q[t, 2 * h + m]) * scale, dim=0) @ vals[:, h // g, :] for m in range(2)]
                o = a[0] - lam * a[1]
                o = out_scale * o * torch.rsqrt((o * o).mean() + sub_eps)
            out[t, out_col + h * v_dim:out_col + (h + 1) * v_dim] = o.to(out.dtype)


def _turned(x, frequencies, positions):
    if frequencies is not None and frequencies.numel():
        half = frequencies.numel()
        ang = positions.float()[:, None] * frequencies.float()[None, :]
        c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
        a, b = x[..., :half].clone(), x[..., half:2 * half].clone()
        x[..., :half] = a * c - b * s
        x[..., half:2 * half] = b * c + a * s
    return x


def retention_carry(state, ends, starts, seq_row, seq_first, seq_count, seg_len, decay, status=None):
    for s in range(seq_row.numel()):
        row, first, count = int(seq_row[s]), int(seq_first[s]), int(seq_count[s])
        S = state[row].clone()
        for j in range(first, first + count):
            starts[j] = S
            S = (decay ** int(seg_len[j]))[:, None, None] * S + ends[j]
        state[row] = S


def _silu(x):
    return x / (1.0 + torch.exp(-x))


def retention_fix(y, q_col, positions, frequencies, starts, tiles, decay, o, act=0):
    heads, dim, v_dim = starts.shape[1:]
    q = y[:, q_col:q_col + heads * dim].float().view(-1, heads, dim).clone()
    q = _turned(_silu(q) if act else q, frequencies, positions)
    for seg, begin, n, t0 in tiles.tolist():
        for t in range(begin, begin + n):
            add = torch.einsum("hdv,hd->hv", starts[seg], q[t]) * (decay ** (t - t0 + 1))[:, None]
            o[t] += add.reshape(-1)


def retention_scan(y, q_col, k_col, v_col, decay, k_scale, frequencies, positions, state, cu_q, rows, o, heads, dim, v_dim,
                   status=None, most_threads=0, ends=None, act=0):
    yf = y.float()
    T = y.shape[0]
    if act:                                      # q, k and v pass through silu as they are read
        yf = yf.clone()
        for col, n in ((q_col, heads * dim), (k_col, heads * dim), (v_col, heads * v_dim)):
            yf[:, col:col + n] = _silu(yf[:, col:col + n])

    def turn(x):
        if frequencies is not None and frequencies.numel():
            half = frequencies.numel()
            ang = positions.float()[:, None] * frequencies.float()[None, :]
            c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
            a, b = x[..., :half].clone(), x[..., half:2 * half].clone()
            x[..., :half] = a * c - b * s
            x[..., half:2 * half] = b * c + a * s
        return x

    q = turn(yf[:, q_col:q_col + heads * dim].view(T, heads, dim).clone())
    k = turn(yf[:, k_col:k_col + heads * dim].view(T, heads, dim).clone()) * k_scale
    v = yf[:, v_col:v_col + heads * v_dim].view(T, heads, v_dim)
    for row, a, b in _sequences(cu_q, rows):
        S = torch.zeros_like(state[0]) if row < 0 else state[row].clone()      # a later segment of a cut walk starts from zeros
        for t in range(a, b):
            S = decay[:, None, None] * S + k[t][:, :, None] * v[t][:, None, :]
            o[t] = torch.einsum("hdv,hd->hv", S, q[t]).reshape(-1)
        if row < 0:
            ends[-row - 1] = S
        else:
            state[row] = S


def _pick_weights(z, mode, scale):
    if mode == 0:
        return torch.softmax(z, dim=0)
    s = torch.sigmoid(z)
    return s / (s.sum() + 1e-20) * scale


def route_experts(logits, top, act, inter, x=None, router=None, mode=0, scale=1.0):
    if logits is None:
        logits = x.float() @ router.float().t()
    T, n = logits.shape
    w = torch.zeros((T, n), dtype=torch.float32)
    chosen = torch.zeros((T, n), dtype=torch.bool)
    for t in range(T):
        order = sorted(range(n), key=lambda e: (-float(logits[t, e]), e))[:top]
        w[t, order] = _pick_weights(logits[t, order], mode, scale)
        chosen[t, order] = True
    scaled = act[:, :n * inter].float().view(T, n, inter) * w[:, :, None]
    act[:, :n * inter] = torch.where(chosen[:, :, None], scaled, torch.zeros_like(scaled)).reshape(T, n * inter).to(act.dtype)


def route_topk(logits, top, ids, weights, x=None, router=None, mode=0, scale=1.0):
    if logits is None:
        logits = x.float() @ router.float().t()
    for t in range(logits.shape[0]):
        order = sorted(range(logits.shape[1]), key=lambda e: (-float(logits[t, e]), e))[:top]
        ids[t] = torch.tensor(order, dtype=torch.int32)
        weights[t] = _pick_weights(logits[t, order], mode, scale)


def expert_lists(ids, lists, counts):
    flat = ids.reshape(-1)
    for e in range(lists.shape[0]):
        mine = torch.nonzero(flat == e).flatten().to(torch.int32)
        lists[e, :mine.numel()] = mine
        counts[e] = mine.numel()


def gather_picks(x, lists, counts, top, rows, where):
    r = 0
    for e in range(lists.shape[0]):
        for i in range(int(counts[e])):
            pick = int(lists[e, i])
            rows[r] = x[pick // top]
            where[pick] = r
            r += 1


def combine_picks(y, where, weights, shared_y, out):
    T, top = weights.shape
    acc = (weights[:, :, None] * y[where.long()].float().view(T, top, -1)).sum(dim=1)
    if shared_y is not None:
        acc = acc + shared_y.float()
    out.copy_(acc.to(out.dtype))


# ---- the kernels of layers with a latent for each token ----


def token_shift(x, mu, state, cu_q, rows, token_seq, out, status=None):
    out.zero_()
    for row, a, b in _sequences(cu_q, rows):
        before = torch.cat([state[row][None], x[a:b - 1]], dim=0)
        out[a:b] = (x[a:b] + (before - x[a:b]) * mu).to(out.dtype)
        state[row] = x[b - 1]


def _turn_pairs(v, positions, frequencies, mult):
    """v [T, ..., n] float: the first 2 * len(frequencies) numbers in pairs (2i, 2i + 1) turned by position * frequencies[i]."""
    if frequencies is None or not frequencies.numel():
        return v
    n = 2 * frequencies.numel()
    ang = positions.float()[:, None] * frequencies.float()[None, :]
    shape = [v.shape[0]] + [1] * (v.dim() - 2) + [frequencies.numel()]
    c, s = (torch.cos(ang) * mult).reshape(shape), (torch.sin(ang) * mult).reshape(shape)
    a, b = v[..., 0:n:2].clone(), v[..., 1:n:2].clone()
    v = v.clone()
    v[..., 0:n:2] = a * c - b * s
    v[..., 1:n:2] = b * c + a * s
    return v


def latent_prepare(y, q_col, q_rank, kv_col, kv_rank, rot_dim, q_weight, k_weight, eps, frequencies, mult, positions, token_seq,
                   block_table, cq, pages, store=True, status=None):
    yf = y.float()
    live = token_seq >= 0
    norm = lambda v, w: v * torch.rsqrt((v * v).mean(dim=-1, keepdim=True) + eps) * w
    cq[live, :q_rank] = norm(yf[:, q_col:q_col + q_rank], q_weight)[live].to(cq.dtype)
    if not store:
        return
    c = norm(yf[:, kv_col:kv_col + kv_rank], k_weight)
    r = _turn_pairs(yf[:, kv_col + kv_rank:kv_col + kv_rank + rot_dim], positions, frequencies, mult)
    row = torch.cat([c, r], dim=-1).to(pages.dtype)
    page_size = pages.shape[2]
    for t in range(y.shape[0]):
        if not bool(live[t]):
            continue
        p = int(positions[t])
        page = int(block_table[int(token_seq[t]), p // page_size])
        assert page >= 0, "a latent is stored into a page that is not held"
        pages[page, 0, p % page_size, :] = row[t]


def head_matmul(x, x_col, x_head, m, out, out_col, out_head, mode=0, tail=0, frequencies=None, mult=1.0, positions=None,
                token_seq=None, gate=None, gate_col=0):
    heads, inner, outer = m.shape
    xf = x.float()
    for h in range(heads):
        a = xf[:, x_col + h * x_head:x_col + h * x_head + inner]
        v = a @ m[h].float()
        if mode == 2 and gate is not None:
            v = v * torch.sigmoid(gate[:, gate_col + h * outer:gate_col + (h + 1) * outer].float())
        out[:, out_col + h * out_head:out_col + h * out_head + outer] = v.to(out.dtype)
        if mode == 1 and tail:
            r = xf[:, x_col + h * x_head + inner:x_col + h * x_head + inner + tail]
            turned = _turn_pairs(r, positions.clamp(min=0), frequencies, mult)
            live = (token_seq >= 0)[:, None]
            out[:, out_col + h * out_head + outer:out_col + h * out_head + outer + tail] = torch.where(live, turned, r).to(out.dtype)


def xielu(z, out, ap, an):
    v = z.float()
    out.copy_(torch.where(v > 0, ap * v * v + 0.5 * v, an * (torch.expm1(v.clamp(max=0.0)) - v) + 0.5 * v).to(out.dtype))


def gate_clamp(gu, out, interleave, alpha, limit, split, limit2):
    inter = out.shape[1]
    if interleave:
        pairs = gu.view(gu.shape[0], inter // 8, 2, 8).float()
        g, u = pairs[:, :, 0].reshape(-1, inter), pairs[:, :, 1].reshape(-1, inter)
    else:
        g, u = gu[:, :inter].float(), gu[:, inter:].float()
    lim = torch.where(torch.arange(inter) >= split, torch.tensor(float(limit2)), torch.tensor(float(limit)))
    g = torch.minimum(g, lim)
    u = torch.maximum(torch.minimum(u, lim), -lim)
    out.copy_((g * torch.sigmoid(alpha * g) * (u + 1.0)).to(out.dtype))


# ---- the kernels of the delta rule with one decay a head, the matrix memory, and mixers whose results are normed and added ----


def _conv_inputs(y, col, width, tail, tail_at, row, a, b):
    """The inputs of a convolution for the step's tokens [a, b) of a request, with the kept inputs in front of them."""
    x = y[a:b, col:col + width].float()
    if tail is None:
        return x
    return torch.cat([tail[row][:, tail_at:tail_at + width], x], dim=0)


def gated_delta_scan(y, q_col, k_col, v_col, b_col, a_col, conv_q, conv_k, conv_v, a_log, dt_bias, key_eps, q_scale, state, tail,
                     cu_q, rows, o, heads, kv_heads, dim, v_dim, status=None, most_threads=0):
    yf = y.float()
    nq, nv = kv_heads * dim, heads * v_dim
    group = heads // kv_heads
    for row, a, b in _sequences(cu_q, rows):
        n = b - a
        made = []
        for col, width, w, at in ((q_col, nq, conv_q, 0), (k_col, nq, conv_k, nq), (v_col, nv, conv_v, 2 * nq)):
            x = _conv_inputs(yf, col, width, tail, at, row, a, b)
            if w is None:
                z = x[-n:]
            else:
                taps = w.shape[1]
                if x.shape[0] < n + taps - 1:
                    x = torch.cat([torch.zeros((n + taps - 1 - x.shape[0], width)), x], dim=0)
                z = sum(x[j:j + n] * w[:, j][None, :] for j in range(taps))
            made.append(z * torch.sigmoid(z))
        q, k, v = made[0].view(n, kv_heads, dim), made[1].view(n, kv_heads, dim), made[2].view(n, heads, v_dim)
        q = q * torch.rsqrt((q * q).sum(dim=-1, keepdim=True) + key_eps) * q_scale
        k = k * torch.rsqrt((k * k).sum(dim=-1, keepdim=True) + key_eps)
        beta = torch.sigmoid(yf[a:b, b_col:b_col + heads])
        decay = torch.exp(-torch.exp(a_log) * torch.nn.functional.softplus(yf[a:b, a_col:a_col + heads] + dt_bias))
        S = state[row].clone()
        for t in range(n):
            kk, qq = k[t].repeat_interleave(group, dim=0), q[t].repeat_interleave(group, dim=0)
            S = decay[t][:, None, None] * S
            u = beta[t][:, None] * (v[t] - torch.einsum("hdv,hd->hv", S, kk))
            S = S + kk[:, :, None] * u[:, None, :]
            o[a + t] = torch.einsum("hdv,hd->hv", S, qq).reshape(-1)
        state[row] = S


def conv_tail_update(y, cols, widths, tail, cu_q, rows, status=None):
    keep = tail.shape[1]
    for row, a, b in _sequences(cu_q, rows):
        x = torch.cat([y[a:b, c:c + w].float() for c, w in zip(cols, widths)], dim=1)
        tail[row] = torch.cat([tail[row], x], dim=0)[-keep:]


def memory_scan(y, q_col, k_col, v_col, i_col, f_col, i_bias, f_bias, gate_cap, q_scale, den_eps, state, cu_q, rows, o, heads, dim,
                v_dim, status=None, most_threads=0):
    yf = y.float()
    T = y.shape[0]
    q = yf[:, q_col:q_col + heads * dim].view(T, heads, dim) * q_scale
    k = yf[:, k_col:k_col + heads * dim].view(T, heads, dim)
    v = yf[:, v_col:v_col + heads * v_dim].view(T, heads, v_dim)
    ig = gate_cap * torch.tanh((yf[:, i_col:i_col + heads] + i_bias) / gate_cap)
    fg = torch.nn.functional.logsigmoid(gate_cap * torch.tanh((yf[:, f_col:f_col + heads] + f_bias) / gate_cap))
    for row, a, b in _sequences(cu_q, rows):
        S, n, m = state[row, :, :dim, :v_dim].clone(), state[row, :, :dim, v_dim].clone(), state[row, :, dim, 0].clone()
        for t in range(a, b):
            m_new = torch.maximum(fg[t] + m, ig[t])
            keep, take = torch.exp(fg[t] + m - m_new), torch.exp(ig[t] - m_new)
            S = keep[:, None, None] * S + take[:, None, None] * k[t][:, :, None] * v[t][:, None, :]
            n = keep[:, None] * n + take[:, None] * k[t]
            m = m_new
            den = torch.maximum((n * q[t]).sum(dim=-1).abs(), torch.exp(-m)) + den_eps
            o[t] = (torch.einsum("hdv,hd->hv", S, q[t]) / den[:, None]).reshape(-1)
        state[row, :, :dim, :v_dim], state[row, :, :dim, v_dim], state[row, :, dim, 0] = S, n, m


def normed_sum(parts, weights, eps, scales, out):
    total = torch.zeros_like(out)
    for p, w, c in zip(parts, weights, scales):
        total = total + c * w * p * torch.rsqrt((p * p).mean(dim=-1, keepdim=True) + eps)
    out.copy_(total)


def add_rows(x, other):
    x.add_(other)


def gate_into(src, y, gate_col, mode, dst, dst_col, scale, heads, v_dim):
    v = src.float().view(src.shape[0], heads, v_dim) * scale
    if mode == 1:
        v = v * torch.sigmoid(y[:, gate_col:gate_col + heads].float())[:, :, None]
    elif mode == 2:
        v = v * torch.sigmoid(y[:, gate_col:gate_col + heads * v_dim].float()).view(-1, heads, v_dim)
    dst[:, dst_col:dst_col + heads * v_dim] = v.reshape(src.shape[0], -1).to(dst.dtype)
