// The general attention: values of another size than keys, a rotation of the first dimensions of a head only with
// the angle formed where it is used, q and k divided by their root mean square after the rotation, and a mask of
// chunks beside the causal one and the window, first tokens that stay visible beside a window, a norm of q and k with a
// weight before the rotation, and two maps of queries and keys a head over one set of values whose results are
// subtracted and normed (differential attention); a norm of q and of k over all their heads together, a query
// temperature that grows with the position, capped scores, a sink in the denominator and a gate on a head's result.
//
// Two kernels.  `attention_prepare` (one block a token, one warp a head): rotation of pairs (i, i + half) by
// position * frequency[i] (a 32-bit product, precise sine and cosine), the norm over the head in 32-bit, q written
// back in place, k and v stored into their pages.  `attention_general` (one warp for a (token, head)): the visible
// keys one after the other in the order of their positions with a running maximum and sum in 32-bit, as in the plain
// attention kernel, so that a token's result depends on its own keys only.
#include "common.cuh"
#include "kernels.h"
#include "launch.cuh"

namespace vtb {

namespace {
constexpr int kMaxPerLane = 8;       // head sizes up to 256
constexpr int kWidePerLane = 32;     // values of up to 1,024 numbers for the attention of one map
constexpr int kPrepareWarps = 8;
}

template <typename T>
__global__ void __launch_bounds__(32 * kPrepareWarps)
attention_prepare_kernel(T* __restrict__ y, int stride, int q_col, int k_col, int v_col, const int* __restrict__ positions,
                         const int* __restrict__ token_seq, const float* __restrict__ freq, int half, float norm_eps,
                         T* __restrict__ k_cache, T* __restrict__ v_cache, const int* __restrict__ block_table,
                         int table_stride, int n_seqs, int n_pages, int heads, int kv_heads, int dim, int v_dim,
                         int page_size, int store, int* status, int v_heads, const float* __restrict__ q_weight,
                         const float* __restrict__ k_weight, int norm_first, int whole, float rot_mult, float qt_coef, int qt_every) {
    __shared__ float head[kPrepareWarps][32 * kMaxPerLane];
    __shared__ float scratch[32];
    pdl_launch();
    const int t = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int seq = token_seq[t];
    const bool seq_ok = seq >= 0 && seq < n_seqs;
    const int pos = seq_ok ? positions[t] : 0;
    const int page = (store && seq_ok && pos >= 0) ? block_table[(size_t)seq * table_stride + pos / page_size] : 0;
    pdl_wait();
    if (seq < 0) return;   // padding
    if (!seq_ok) {
        if (threadIdx.x == 0) set_status(status, kStatusBadSequence, seq);
        return;
    }
    if (pos < 0) {
        if (threadIdx.x == 0) set_status(status, kStatusBadPosition, pos);
        return;
    }
    if (store && (page < 0 || page >= n_pages)) {
        if (threadIdx.x == 0) set_status(status, kStatusBadPage, page);
        store = 0;
    }
    T* row = y + (size_t)t * stride;
    const int slot = pos % page_size;
    const int units = heads + (store ? kv_heads : 0);
    float* hv = head[warp];
    // the norm over the whole projection: one mean square over all heads of q, one over all heads of k (the block is
    // one token's, so every thread is here)
    float whole_q = 1.f, whole_k = 1.f;
    if (whole && norm_eps >= 0.f) {
        float sq = 0.f, sk = 0.f;
        for (int e = threadIdx.x; e < heads * dim; e += blockDim.x) { const float v = to_float(row[q_col + e]); sq = fmaf(v, v, sq); }
        for (int e = threadIdx.x; e < kv_heads * dim; e += blockDim.x) { const float v = to_float(row[k_col + e]); sk = fmaf(v, v, sk); }
        whole_q = rsqrtf(block_sum(sq, scratch) / (float)(heads * dim) + norm_eps);
        whole_k = rsqrtf(block_sum(sk, scratch) / (float)(kv_heads * dim) + norm_eps);
    }
    // the query's temperature: 1 + c ln(floor((p + 1) / n) + 1)
    const float q_times = qt_coef != 0.f ? 1.f + qt_coef * logf((float)((pos + 1) / qt_every) + 1.f) : 1.f;
    // (a step of few tokens is cut over gridDim.y blocks a token: each takes every gridDim.y-th group of heads)
    for (int u = warp + kPrepareWarps * blockIdx.y; u < units; u += kPrepareWarps * gridDim.y) {
        const bool is_q = u < heads;
        T* src = is_q ? row + q_col + u * dim : row + k_col + (u - heads) * dim;
        for (int i = lane; i < dim; i += 32) hv[i] = to_float(src[i]);
        __syncwarp();
        const float* w = is_q ? q_weight : k_weight;           // the norm's weight [dim] (or none); [all heads * dim] with whole
        if (whole && norm_eps >= 0.f) {
            const float sc = is_q ? whole_q : whole_k;
            const float* wh = w ? w + (size_t)(is_q ? u : u - heads) * dim : nullptr;
            for (int i = lane; i < dim; i += 32) hv[i] = hv[i] * sc * (wh ? wh[i] : 1.f);
            __syncwarp();
        } else if (norm_first && norm_eps >= 0.f) {
            // the norm comes before the rotation: the head is normed where it lies, then turned
            float s0 = 0.f;
            for (int i = lane; i < dim; i += 32) s0 = fmaf(hv[i], hv[i], s0);
            const float sc = rsqrtf(warp_sum(s0) / (float)dim + norm_eps);
            for (int i = lane; i < dim; i += 32) hv[i] = hv[i] * sc * (w ? w[i] : 1.f);
            __syncwarp();
        }
        float x[kMaxPerLane];
        float ss = 0.f;
#pragma unroll
        for (int r = 0; r < kMaxPerLane; ++r) {
            const int i = lane + 32 * r;
            float v = 0.f;
            if (i < dim) {
                v = hv[i];
                if (i < 2 * half) {
                    const int f = i < half ? i : i - half;
                    const float angle = (float)pos * freq[f];
                    float sn, cs;
                    sincosf(angle, &sn, &cs);
                    sn *= rot_mult;
                    cs *= rot_mult;
                    v = i < half ? v * cs - hv[i + half] * sn : v * cs + hv[i - half] * sn;
                }
            }
            x[r] = v;
            ss = fmaf(v, v, ss);
        }
        float scale = 1.f;
        const bool after = !norm_first && !whole && norm_eps >= 0.f;
        if (after) scale = rsqrtf(warp_sum(ss) / (float)dim + norm_eps);
        if (is_q) scale *= q_times;
        T* dst = is_q ? src : k_cache + (((size_t)page * kv_heads + (u - heads)) * page_size + slot) * dim;
#pragma unroll
        for (int r = 0; r < kMaxPerLane; ++r) {
            const int i = lane + 32 * r;
            if (i < dim) dst[i] = from_float<T>(x[r] * scale * ((after && w) ? w[i] : 1.f));
        }
        __syncwarp();
    }
    if (!store) return;
    for (int e = threadIdx.x + blockIdx.y * blockDim.x; e < v_heads * v_dim; e += blockDim.x * gridDim.y) {
        const int h = e / v_dim, i = e % v_dim;
        v_cache[(((size_t)page * v_heads + h) * page_size + slot) * v_dim + i] = row[v_col + e];
    }
}

cudaError_t launch_attention_prepare(int dtype, void* y, int stride, int q_col, int k_col, int v_col, const int* positions,
                                     const int* token_seq, const float* freq, int half, float norm_eps, void* k_cache,
                                     void* v_cache, const int* block_table, int table_stride, int n_seqs, int n_pages,
                                     int n_tokens, int heads, int kv_heads, int dim, int v_dim, int page_size, int store,
                                     int* status, int v_heads, const float* q_weight, const float* k_weight, int norm_first,
                                     cudaStream_t stream, int whole, float rot_mult, float qt_coef, int qt_every) {
    if (n_tokens == 0) return cudaSuccess;
    if (qt_every < 1) return cudaErrorInvalidValue;
    if (dim > 32 * kMaxPerLane || 2 * half > dim) return cudaErrorInvalidValue;
    // few tokens: several blocks a token, so that a step of single tokens fills the SMs (not with the norm over the whole
    // projection: a block would write a head of q back while another still adds up the squares of all of them)
    const int slices = (n_tokens >= 1024 || whole) ? 1 : max(1, min(8, (heads + kv_heads + 2 * kPrepareWarps - 1) / (2 * kPrepareWarps)));
    const dim3 grid(n_tokens, slices);
    if (dtype == kBF16)
        return launch(attention_prepare_kernel<__nv_bfloat16>, grid, 32 * kPrepareWarps, 0, stream, (__nv_bfloat16*)y, stride,
                      q_col, k_col, v_col, positions, token_seq, freq, half, norm_eps, (__nv_bfloat16*)k_cache,
                      (__nv_bfloat16*)v_cache, block_table, table_stride, n_seqs, n_pages, heads, kv_heads, dim, v_dim,
                      page_size, store, status, v_heads, q_weight, k_weight, norm_first, whole, rot_mult, qt_coef, qt_every);
    return launch(attention_prepare_kernel<float>, grid, 32 * kPrepareWarps, 0, stream, (float*)y, stride, q_col, k_col,
                  v_col, positions, token_seq, freq, half, norm_eps, (float*)k_cache, (float*)v_cache, block_table,
                  table_stride, n_seqs, n_pages, heads, kv_heads, dim, v_dim, page_size, store, status, v_heads, q_weight, k_weight,
                  norm_first, whole, rot_mult, qt_coef, qt_every);
}

// One warp for a (token, head).  The visible keys are taken 32 at a time, a lane a key: the lane forms its key's whole
// score from q in shared memory (no exchange between lanes for a score), the block's maximum and sum are found once,
// and the block's values are added with a lane owning dimensions i, i + 32, ... of the result.  The blocks start at the
// first visible key, which depends on the token's position alone, so a token's result does not depend on the step.
// With a window and `keep_first`, the keys at positions below keep_first that the window has passed come first, in
// blocks that start at key 0.  MAPS 2: the head has two queries and its head of values two heads of keys; a lane forms
// both scores of its key, each map keeps a maximum, a sum and a result of its own over the same values (read once),
// and the end is o = a_1 - lam a_2, divided by its root mean square.
// `sinks` [heads] (or null): one more term exp(sinks[h]) in the softmax's denominator, without a key or a value and not
// scaled.  `v_stride`: elements from one value row to the next in `v_cache` (v_dim where the values have pages of their own;
// the key's size where a value is the first v_dim numbers of its key's row and `v_cache` is `k_cache`).  PL: values of a
// head that a lane holds (head sizes up to 32 PL); the queries lie in dynamic shared memory.
template <typename T, bool Vec, int MAPS, int PL>
__global__ void __launch_bounds__(128)
attention_general_kernel(const T* __restrict__ y, int stride, int q_col, T* __restrict__ out, int out_stride, int out_col,
                         float out_scale, const T* __restrict__ k_cache, const T* __restrict__ v_cache,
                         const int* __restrict__ positions, const int* __restrict__ token_seq,
                         const int* __restrict__ block_table, int table_stride, int n_seqs, int n_pages, int n_tokens,
                         int heads, int kv_heads, int dim, int v_dim, int page_size, int window, int chunk, float scale,
                         int* status, int keep_first, float lam, float sub_eps, const float* __restrict__ sinks, int v_stride,
                         float softcap, int gate_mode, int gate_col) {
    extern __shared__ __align__(16) float qs_all[];
    constexpr int kMaxPerLane = PL;
    pdl_launch();
    pdl_wait();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const long long pair = (long long)blockIdx.x * (blockDim.x >> 5) + warp;
    if (pair >= (long long)n_tokens * heads) return;
    const int t = (int)(pair / heads), h = (int)(pair % heads);
    const int seq = token_seq[t];
    T* o = out + (size_t)t * out_stride + out_col + (size_t)h * v_dim;
    if (seq < 0) {   // padding
        for (int i = lane; i < v_dim; i += 32) o[i] = from_float<T>(0.f);
        return;
    }
    if (seq >= n_seqs) {
        if (lane == 0) set_status(status, kStatusBadSequence, seq);
        return;
    }
    const int pos = positions[t];
    const int kvh = h / (heads / kv_heads);
    const int* table = block_table + (size_t)seq * table_stride;
    const int dim_s = (dim + 3) & ~3;                              // a map's query starts on a 16-byte boundary
    float* q = qs_all + warp * MAPS * dim_s;
    const T* qp = y + (size_t)t * stride + q_col + (size_t)h * MAPS * dim;
    for (int i = lane; i < MAPS * dim; i += 32) q[(i / dim) * dim_s + i % dim] = to_float(qp[i]) * scale;
    __syncwarp();

    float acc[MAPS][kMaxPerLane];
    float mx[MAPS], sum[MAPS];
#pragma unroll
    for (int m = 0; m < MAPS; ++m) {
        mx[m] = -INFINITY;
        sum[m] = 0.f;
#pragma unroll
        for (int r = 0; r < kMaxPerLane; ++r) acc[m][r] = 0.f;
    }
    const int first = first_visible_key(pos, window, chunk);
    // the kept first tokens that the window has passed (none without a window, and none beside chunks)
    const int kept = (window > 0 && chunk <= 0) ? min(keep_first, first) : 0;
    for (int part = 0; part < 2; ++part) {
        const int lo = part == 0 ? 0 : first, hi = part == 0 ? kept : pos + 1;
        for (int j0 = lo; j0 < hi; j0 += 32) {
            const int j = j0 + lane;
            bool live = j < hi;
            int at_k = 0, at_v = 0;                                // the key's (map 0) and the value's row in the pages
            if (live) {
                const int page = table[j / page_size];
                if (page < 0 || page >= n_pages) {
                    set_status(status, kStatusBadPage, page);
                    live = false;
                } else {
                    at_k = (page * kv_heads * MAPS + kvh * MAPS) * page_size + (j % page_size);
                    at_v = (page * kv_heads + kvh) * page_size + (j % page_size);
                }
            }
            float s[MAPS];
#pragma unroll
            for (int m = 0; m < MAPS; ++m) {
                s[m] = -INFINITY;
                if (!live) continue;
                const T* kp = k_cache + (size_t)(at_k + m * page_size) * dim;
                const float* qm = q + m * dim_s;
                float part4[4] = {0.f, 0.f, 0.f, 0.f};
                if (Vec) {
                    for (int i = 0; i < dim; i += 8) {
                        float k8[8];
                        Vec8<T>::load(kp + i, k8);
                        const float4 qa = *reinterpret_cast<const float4*>(qm + i), qb = *reinterpret_cast<const float4*>(qm + i + 4);
                        part4[0] = fmaf(qa.x, k8[0], part4[0]); part4[1] = fmaf(qa.y, k8[1], part4[1]);
                        part4[2] = fmaf(qa.z, k8[2], part4[2]); part4[3] = fmaf(qa.w, k8[3], part4[3]);
                        part4[0] = fmaf(qb.x, k8[4], part4[0]); part4[1] = fmaf(qb.y, k8[5], part4[1]);
                        part4[2] = fmaf(qb.z, k8[6], part4[2]); part4[3] = fmaf(qb.w, k8[7], part4[3]);
                    }
                } else {
                    for (int i = 0; i < dim; ++i) part4[i & 3] = fmaf(qm[i], to_float(kp[i]), part4[i & 3]);
                }
                s[m] = (part4[0] + part4[1]) + (part4[2] + part4[3]);
                if (softcap > 0.f) s[m] = softcap * tanhf(s[m] / softcap);
            }
            float p[MAPS];
#pragma unroll
            for (int m = 0; m < MAPS; ++m) {
                const float new_mx = fmaxf(mx[m], warp_max(s[m]));     // a block holds at least one visible key: finite
                const float corr = expf(mx[m] - new_mx);               // 0 at the first block (mx = -inf)
                p[m] = live ? expf(s[m] - new_mx) : 0.f;
                sum[m] = sum[m] * corr + warp_sum(p[m]);
                mx[m] = new_mx;
#pragma unroll
                for (int r = 0; r < kMaxPerLane; ++r) acc[m][r] *= corr;
            }
            const int n = min(32, hi - j0);
            for (int jj = 0; jj < n; ++jj) {
                float pj[MAPS];
#pragma unroll
                for (int m = 0; m < MAPS; ++m) pj[m] = __shfl_sync(0xffffffffu, p[m], jj);
                const int aj = __shfl_sync(0xffffffffu, at_v, jj);
                const T* vp = v_cache + (size_t)aj * v_stride;
#pragma unroll
                for (int r = 0; r < kMaxPerLane; ++r) {
                    const int i = lane + 32 * r;
                    if (i < v_dim) {
                        const float v = to_float(vp[i]);
#pragma unroll
                        for (int m = 0; m < MAPS; ++m) acc[m][r] = fmaf(pj[m], v, acc[m][r]);
                    }
                }
            }
        }
    }
    if (MAPS == 1) {
        float den = sum[0], keep = 1.f;
        if (sinks != nullptr) {
            const float sk = sinks[h], top = fmaxf(mx[0], sk);      // the sink may be the largest term
            keep = expf(mx[0] - top);
            den = sum[0] * keep + expf(sk - top);
        }
        float inv = den > 0.f ? out_scale * keep / den : 0.f;
        // the gate on the head's result: one number a head, or one an element, sigmoid of a column of y
        const T* gp = y + (size_t)t * stride + gate_col;
        if (gate_mode == 1) inv *= 1.f / (1.f + expf(-to_float(gp[h])));
#pragma unroll
        for (int r = 0; r < kMaxPerLane; ++r) {
            const int i = lane + 32 * r;
            if (i < v_dim) {
                float v = acc[0][r] * inv;
                if (gate_mode == 2) v *= 1.f / (1.f + expf(-to_float(gp[(size_t)h * v_dim + i])));
                o[i] = from_float<T>(v);
            }
        }
        return;
    }
    // the difference of the two maps, divided by its root mean square over the head's values
    const float inv0 = sum[0] > 0.f ? 1.f / sum[0] : 0.f;
    const float inv1 = sum[MAPS - 1] > 0.f ? 1.f / sum[MAPS - 1] : 0.f;
    float d[kMaxPerLane];
    float ss = 0.f;
#pragma unroll
    for (int r = 0; r < kMaxPerLane; ++r) {
        const int i = lane + 32 * r;
        d[r] = i < v_dim ? acc[0][r] * inv0 - lam * (acc[MAPS - 1][r] * inv1) : 0.f;
        ss = fmaf(d[r], d[r], ss);
    }
    const float rs = rsqrtf(warp_sum(ss) / (float)v_dim + sub_eps) * out_scale;
#pragma unroll
    for (int r = 0; r < kMaxPerLane; ++r) {
        const int i = lane + 32 * r;
        if (i < v_dim) o[i] = from_float<T>(d[r] * rs);
    }
}

template <typename T>
static cudaError_t launch_attention_general_t(const T* y, int stride, int q_col, T* out, int out_stride, int out_col, float out_scale,
                                              const T* k_cache, const T* v_cache, const int* positions, const int* token_seq,
                                              const int* block_table, int table_stride, int n_seqs, int n_pages, int n_tokens,
                                              int heads, int kv_heads, int dim, int v_dim, int page_size, int window, int chunk,
                                              float scale, int* status, int keep_first, int maps, float lam, float sub_eps,
                                              const float* sinks, int v_stride, cudaStream_t stream, float softcap, int gate_mode,
                                              int gate_col) {
    const long long pairs = (long long)n_tokens * heads;
    const int blocks = (int)((pairs + 3) / 4);
    // a key's row is read in 16-byte pieces where every row starts on such a boundary
    const bool vec = dim % 8 == 0 && (reinterpret_cast<uintptr_t>(k_cache) & 15) == 0;
    const bool wide = v_dim > 32 * kMaxPerLane;                     // one map with values of up to 32 * kWidePerLane numbers
    auto kernel = maps == 2 ? (vec ? attention_general_kernel<T, true, 2, kMaxPerLane> : attention_general_kernel<T, false, 2, kMaxPerLane>)
                  : wide    ? (vec ? attention_general_kernel<T, true, 1, kWidePerLane> : attention_general_kernel<T, false, 1, kWidePerLane>)
                            : (vec ? attention_general_kernel<T, true, 1, kMaxPerLane> : attention_general_kernel<T, false, 1, kMaxPerLane>);
    const size_t bytes = (size_t)4 * maps * ((dim + 3) & ~3) * sizeof(float);
    return launch(kernel, blocks, 128, bytes, stream, y, stride, q_col, out, out_stride, out_col, out_scale, k_cache, v_cache, positions,
                  token_seq, block_table, table_stride, n_seqs, n_pages, n_tokens, heads, kv_heads, dim, v_dim, page_size, window,
                  chunk, scale, status, keep_first, lam, sub_eps, sinks, v_stride > 0 ? v_stride : v_dim, softcap, gate_mode, gate_col);
}

cudaError_t launch_attention_general(int dtype, const void* y, int stride, int q_col, void* out, int out_stride, int out_col,
                                     float out_scale, const void* k_cache, const void* v_cache, const int* positions,
                                     const int* token_seq, const int* block_table, int table_stride, int n_seqs, int n_pages,
                                     int n_tokens, int heads, int kv_heads, int dim, int v_dim, int page_size, int window,
                                     int chunk, float scale, int* status, int keep_first, int maps, float lam, float sub_eps,
                                     cudaStream_t stream, const float* sinks, int v_stride, float softcap, int gate_mode,
                                     int gate_col) {
    if (n_tokens == 0) return cudaSuccess;
    if ((softcap > 0.f || gate_mode != 0) && maps != 1) return cudaErrorInvalidValue;
    // keys of any size up to what four queries take of shared memory; values up to 256 numbers (two maps) or 1,024 (one)
    if (dim > 2048 || v_dim > 32 * (maps == 2 ? kMaxPerLane : kWidePerLane) || (maps != 1 && maps != 2)) return cudaErrorInvalidValue;
    if (sinks != nullptr && maps != 1) return cudaErrorInvalidValue;
    if (dtype == kBF16)
        return launch_attention_general_t((const __nv_bfloat16*)y, stride, q_col, (__nv_bfloat16*)out, out_stride, out_col, out_scale,
                                          (const __nv_bfloat16*)k_cache, (const __nv_bfloat16*)v_cache, positions, token_seq,
                                          block_table, table_stride, n_seqs, n_pages, n_tokens, heads, kv_heads, dim, v_dim,
                                          page_size, window, chunk, scale, status, keep_first, maps, lam, sub_eps, sinks, v_stride, stream,
                                          softcap, gate_mode, gate_col);
    return launch_attention_general_t((const float*)y, stride, q_col, (float*)out, out_stride, out_col, out_scale, (const float*)k_cache,
                                      (const float*)v_cache, positions, token_seq, block_table, table_stride, n_seqs, n_pages,
                                      n_tokens, heads, kv_heads, dim, v_dim, page_size, window, chunk, scale, status, keep_first,
                                      maps, lam, sub_eps, sinks, v_stride, stream, softcap, gate_mode, gate_col);
}

}  // namespace vtb
