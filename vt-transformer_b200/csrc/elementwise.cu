// Embedding, RMS norm with the residual sum, SiLU * up, rotation with the cache store.
//
// Formulas after vt-transformer's kernels: v1/tensortype/cuda_kernels/rmsnorm.cu:20-47
// (w * x * rsqrt(mean(x^2) + eps), all in 32-bit, one rounding),
// v1/tensortype/cuda_kernels/rotary_embed.cu:19-29 (pairs (i, i + d/2)),
// v1/tensortype/cuda_kernels/silu_product.cu:15-17 (act / (1 + exp(-act)) * in),
// v1/tensortype/host_tensor.cpp:189-198 (the embedding is a copy of rows).
// The launch shapes are this engine's: one block a token, 16-byte accesses, the residual
// sum folded into the norm, and the keys and values written straight into their pages.
#include "common.cuh"
#include "kernels.h"
#include "launch.cuh"

namespace vtb {

// ------------------------------------------------------------------------- embedding

template <typename T>
__global__ void embedding_kernel(const T* __restrict__ table, const int* __restrict__ ids, float* __restrict__ out,
                                 int hidden, int vocab, float scale, int* status) {
    pdl_launch();
    pdl_wait();
    const int t = blockIdx.x;
    const int id = ids[t];
    float* o = out + (size_t)t * hidden;
    if (id < 0 || id >= vocab) {
        if (threadIdx.x == 0 && id >= vocab) set_status(status, kStatusBadTokenId, id);
        // a negative id marks a padding token: its row is zero
        for (int i = threadIdx.x * 8; i < hidden; i += blockDim.x * 8) {
            float z[8] = {0, 0, 0, 0, 0, 0, 0, 0};
            Vec8<float>::store(o + i, z);
        }
        return;
    }
    const T* row = table + (size_t)id * hidden;
    for (int i = threadIdx.x * 8; i < hidden; i += blockDim.x * 8) {
        float f[8];
        Vec8<T>::load(row + i, f);
        if (scale != 1.0f) {
#pragma unroll
            for (int j = 0; j < 8; ++j) f[j] *= scale;
        }
        Vec8<float>::store(o + i, f);
    }
}

cudaError_t launch_embedding(int table_dtype, const void* table, const int* ids, float* out, int n_tokens,
                             int hidden, int vocab, float scale, int* status, cudaStream_t stream) {
    if (n_tokens == 0) return cudaSuccess;
    int threads = min(256, max(32, ((hidden / 8 + 31) / 32) * 32));
    if (table_dtype == kBF16)
        return launch(embedding_kernel<__nv_bfloat16>, n_tokens, threads, 0, stream, (const __nv_bfloat16*)table, ids, out, hidden, vocab, scale, status);
    return launch(embedding_kernel<float>, n_tokens, threads, 0, stream, (const float*)table, ids, out, hidden, vocab, scale, status);
}

// ------------------------------------------------------------------------- logits: scale and soft cap

// logits = cap * tanh(scale * logits / cap) in place (cap 0: the scale alone), 32-bit.
__global__ void logits_scale_cap_kernel(float* __restrict__ logits, long long n, float scale, float cap) {
    pdl_launch();
    pdl_wait();
    const float inv = cap > 0.f ? 1.f / cap : 0.f;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        float v = logits[i] * scale;
        if (cap > 0.f) v = cap * tanhf(v * inv);
        logits[i] = v;
    }
}

cudaError_t launch_logits_scale_cap(float* logits, long long n, float scale, float cap, cudaStream_t stream) {
    if (n == 0) return cudaSuccess;
    const int blocks = (int)min((n + 255) / 256, (long long)148 * 8);
    return launch(logits_scale_cap_kernel, blocks, 256, 0, stream, logits, n, scale, cap);
}

// ------------------------------------------------------------------------- rmsnorm

// One block a row.  Pass 1 forms v = x (+ delta) in 32-bit, writes it back when there is a
// delta, and sums v^2; pass 2 reads v again (its own writes) and scales it.  The sum's order
// depends on hidden and the block size only, never on the batch.  The delta may also come as `n_parts` 32-bit
// shares [n_parts, n_tokens, hidden] (a matrix product whose inner dimension was cut over CTAs leaves its shares
// unadded): they are added here in the order of their index.
// With `post_weight` the delta is itself normed before it is added: delta * rsqrt(mean(delta^2) + post_eps) * post_weight *
// post_mult, in 32-bit (a layer that norms a sublayer's result before the residual sum): one more pass over the delta's row
// for its sum of squares, whose order depends on hidden and the block size only.
// Groups: a row of `row_size` values is `row_size / hidden` consecutive parts of `hidden` values, each normed by its own
// root mean square (blockIdx.y is the part).  `x_scale` multiplies the stream before the delta is added (v = x_scale x + delta).
// `write_normed`: the stream takes the normed row (in 32-bit) instead of the sum, for a layer whose norm comes after the sum;
// `out` may then be null.
template <typename T, bool Center>
__global__ void rmsnorm_kernel(float* __restrict__ x, const T* __restrict__ delta, const float* __restrict__ parts,
                               int n_parts, const float* __restrict__ weight, float eps, T* __restrict__ out,
                               const int* __restrict__ rows, int n_tokens, int hidden, int* status,
                               const float* __restrict__ post_weight, float post_eps, float post_mult, int row_size,
                               float x_scale, int write_normed) {
    __shared__ float scratch[32];
    pdl_launch();
    // the norm's weight and the list of rows are written by no kernel of the step: they are read before the wait
    const int r = blockIdx.x;
    const int t = rows ? rows[r] : r;
    const int part0 = blockIdx.y * hidden;                   // where this block's part of the row begins
    weight += part0;
    if (post_weight != nullptr) post_weight += part0;
    float w_first[8];
    if ((int)threadIdx.x * 8 < hidden) Vec8<float>::load(weight + threadIdx.x * 8, w_first);
    pdl_wait();
    T* o = out ? out + (size_t)r * row_size + part0 : nullptr;
    if (t < 0 || t >= n_tokens) {
        if (threadIdx.x == 0) set_status(status, kStatusBadRow, t);
        return;
    }
    float* xr = x + (size_t)t * row_size + part0;
    const T* dr = delta ? delta + (size_t)t * row_size + part0 : nullptr;
    const float* pr = parts ? parts + (size_t)t * row_size + part0 : nullptr;
    const size_t stride = (size_t)n_tokens * row_size;
    const int first = threadIdx.x * 8;
    // the delta (a tensor, or the shares in the order of their index) for the eight values at i
    auto delta_values = [&](int i, float (&d)[8]) {
        if (dr) {
            Vec8<T>::load(dr + i, d);
        } else {
#pragma unroll
            for (int j = 0; j < 8; ++j) d[j] = 0.f;
#pragma unroll 4
            for (int q = 0; q < n_parts; ++q) {
                float e[8];
                Vec8<float>::load(pr + i + q * stride, e);
#pragma unroll
                for (int j = 0; j < 8; ++j) d[j] += e[j];
            }
        }
    };
    float post_rs = 0.f;
    if (post_weight != nullptr && (dr || pr)) {
        float ds = 0.f;
        for (int i = first; i < hidden; i += blockDim.x * 8) {
            float d[8];
            delta_values(i, d);
#pragma unroll
            for (int j = 0; j < 8; ++j) ds += d[j] * d[j];
        }
        post_rs = rsqrtf(block_sum(ds, scratch) / (float)hidden + post_eps) * post_mult;
        __syncthreads();                                  // scratch is used again below
    }
    // v = x (+ delta) for the eight values at i
    auto row_values = [&](int i, float (&v)[8]) {
        Vec8<float>::load(xr + i, v);
        if (x_scale != 1.f) {
#pragma unroll
            for (int j = 0; j < 8; ++j) v[j] *= x_scale;
        }
        if (post_weight != nullptr && (dr || pr)) {
            float d[8], w[8];
            delta_values(i, d);
            Vec8<float>::load(post_weight + i, w);
#pragma unroll
            for (int j = 0; j < 8; ++j) v[j] += d[j] * post_rs * w[j];
        } else if (dr) {
            float d[8];
            Vec8<T>::load(dr + i, d);
#pragma unroll
            for (int j = 0; j < 8; ++j) v[j] += d[j];
        } else if (pr) {
#pragma unroll 4
            for (int q = 0; q < n_parts; ++q) {
                float d[8];
                Vec8<float>::load(pr + i + q * stride, d);
#pragma unroll
                for (int j = 0; j < 8; ++j) v[j] += d[j];
            }
        }
    };
    const bool once = hidden <= (int)blockDim.x * 8;      // a thread has all its values at once: they stay in registers
    float keep[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    float ss = 0.f, sm = 0.f;
    for (int i = first; i < hidden; i += blockDim.x * 8) {
        float v[8];
        row_values(i, v);
        if ((dr || pr || x_scale != 1.f) && !(once && write_normed)) Vec8<float>::store(xr + i, v);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            ss += v[j] * v[j];
            sm += v[j];
            keep[j] = v[j];
        }
    }
    float mean = 0.f;
    if (Center) {
        // the layer norm: the mean first, then the mean of the squared deviations from it (not E[v^2] - mean^2)
        mean = block_sum(sm, scratch) / (float)hidden;
        ss = 0.f;
        for (int i = first; i < hidden; i += blockDim.x * 8) {
            float v[8];
            if (once) {
#pragma unroll
                for (int j = 0; j < 8; ++j) v[j] = keep[j];
            } else {
                Vec8<float>::load(xr + i, v);
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) ss += (v[j] - mean) * (v[j] - mean);
        }
    }
    const float total = block_sum(ss, scratch);
    const float rs = rsqrtf(total / (float)hidden + eps);
    for (int i = first; i < hidden; i += blockDim.x * 8) {
        float v[8], w[8], y[8];
        if (once) {
#pragma unroll
            for (int j = 0; j < 8; ++j) v[j] = keep[j];
        } else {
            Vec8<float>::load(xr + i, v);       // its own writes, or x as it was
        }
        if (i == first) {
#pragma unroll
            for (int j = 0; j < 8; ++j) w[j] = w_first[j];
        } else {
            Vec8<float>::load(weight + i, w);
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) y[j] = w[j] * (v[j] - mean) * rs;
        if (o) Vec8<T>::store(o + i, y);
        if (write_normed) Vec8<float>::store(xr + i, y);
    }
}

// Groups of a size that is no multiple of 8 (their rows do not start on 16-byte boundaries): a warp a (row, group), value by
// value; the sum of squares in the order lane by lane, then over the lanes.  No delta that is normed first, no mean.
template <typename T>
__global__ void rmsnorm_narrow_groups_kernel(float* __restrict__ x, const T* __restrict__ delta, const float* __restrict__ parts,
                                             int n_parts, const float* __restrict__ weight, float eps, T* __restrict__ out,
                                             const int* __restrict__ rows, int n_tokens, int part, int* status, int row_size,
                                             float x_scale, int write_normed) {
    pdl_launch();
    const int r = blockIdx.x;
    const int t = rows ? rows[r] : r;
    const int part0 = blockIdx.y * part;
    pdl_wait();
    if (t < 0 || t >= n_tokens) {
        if (threadIdx.x == 0) set_status(status, kStatusBadRow, t);
        return;
    }
    float* xr = x + (size_t)t * row_size + part0;
    const size_t stride = (size_t)n_tokens * row_size;
    float ss = 0.f;
    for (int i = threadIdx.x; i < part; i += 32) {
        float v = xr[i] * x_scale;
        if (delta) v += to_float(delta[(size_t)t * row_size + part0 + i]);
        for (int q = 0; parts && q < n_parts; ++q) v += parts[(size_t)t * row_size + part0 + i + q * stride];
        xr[i] = v;
        ss = fmaf(v, v, ss);
    }
    ss = warp_sum(ss);
    const float rs = rsqrtf(ss / (float)part + eps);
    for (int i = threadIdx.x; i < part; i += 32) {
        const float y = weight[part0 + i] * xr[i] * rs;      // this lane's own write above
        if (out) out[(size_t)r * row_size + part0 + i] = from_float<T>(y);
        if (write_normed) xr[i] = y;
    }
}

template <bool Center>
static cudaError_t launch_norm(int out_dtype, float* x, const void* delta, const float* parts, int n_parts,
                               const float* weight, float eps, void* out, const int* rows, int n_rows, int n_tokens,
                               int hidden, int* status, const float* post_weight, float post_eps, float post_mult,
                               cudaStream_t stream, int groups = 1, float x_scale = 1.f, int write_normed = 0) {
    if (delta != nullptr && parts != nullptr) return cudaErrorInvalidValue;
    if (n_rows == 0) return cudaSuccess;
    if (groups < 1 || hidden % groups || (out == nullptr && !write_normed)) return cudaErrorInvalidValue;
    const int part = hidden / groups;                     // values that are normed together
    if (part % 8) {
        if (Center || post_weight != nullptr) return cudaErrorInvalidValue;
        const dim3 grid_narrow(n_rows, groups);
        if (out_dtype == kBF16)
            return launch(rmsnorm_narrow_groups_kernel<__nv_bfloat16>, grid_narrow, 32, 0, stream, x, (const __nv_bfloat16*)delta, parts, n_parts,
                          weight, eps, (__nv_bfloat16*)out, rows, n_tokens, part, status, hidden, x_scale, write_normed);
        return launch(rmsnorm_narrow_groups_kernel<float>, grid_narrow, 32, 0, stream, x, (const float*)delta, parts, n_parts, weight, eps,
                      (float*)out, rows, n_tokens, part, status, hidden, x_scale, write_normed);
    }
    int threads = min(512, max(32, ((part / 8 + 31) / 32) * 32));
    const dim3 grid(n_rows, groups);
    if (out_dtype == kBF16)
        return launch(rmsnorm_kernel<__nv_bfloat16, Center>, grid, threads, 0, stream, x, (const __nv_bfloat16*)delta, parts, n_parts, weight, eps,
                      (__nv_bfloat16*)out, rows, n_tokens, part, status, post_weight, post_eps, post_mult, hidden, x_scale, write_normed);
    return launch(rmsnorm_kernel<float, Center>, grid, threads, 0, stream, x, (const float*)delta, parts, n_parts, weight, eps, (float*)out, rows, n_tokens,
                  part, status, post_weight, post_eps, post_mult, hidden, x_scale, write_normed);
}

cudaError_t launch_rmsnorm(int out_dtype, float* x, const void* delta, const float* parts, int n_parts,
                           const float* weight, float eps, void* out, const int* rows, int n_rows, int n_tokens,
                           int hidden, int* status, const float* post_weight, float post_eps, float post_mult, cudaStream_t stream,
                           int groups, float x_scale, int write_normed) {
    return launch_norm<false>(out_dtype, x, delta, parts, n_parts, weight, eps, out, rows, n_rows, n_tokens, hidden, status, post_weight,
                       post_eps, post_mult, stream, groups, x_scale, write_normed);
}

cudaError_t launch_layernorm(int out_dtype, float* x, const void* delta, const float* parts, int n_parts,
                             const float* weight, float eps, void* out, const int* rows, int n_rows, int n_tokens,
                             int hidden, int* status, const float* post_weight, float post_eps, float post_mult, cudaStream_t stream) {
    return launch_norm<true>(out_dtype, x, delta, parts, n_parts, weight, eps, out, rows, n_rows, n_tokens, hidden, status, post_weight,
                       post_eps, post_mult, stream);
}

// ------------------------------------------------------------------------- PolyNorm

// One block a row: out = a N(z) + b N(z^2) + c N(z^3) + e with N(y) = y / sqrt(mean(y^2) + eps).  Pass 1 sums z^2,
// z^4 and z^6 in 32-bit (the means are over the first n_mean columns; the others are zero padding); pass 2 reads the row again (each thread the values it read before, so `out` may be `z`).
template <typename T>
__global__ void polynorm_kernel(const T* __restrict__ z, const float* __restrict__ coef, float eps, T* __restrict__ out,
                                int inter, int n_mean) {
    __shared__ float scratch[32];
    pdl_launch();
    const float a = coef[0], b = coef[1], c = coef[2], e = coef[3];      // weights: written by no kernel of the step
    pdl_wait();
    const T* zr = z + (size_t)blockIdx.x * inter;
    T* o = out + (size_t)blockIdx.x * inter;
    float s2 = 0.f, s4 = 0.f, s6 = 0.f;
    for (int i = threadIdx.x * 8; i < inter; i += blockDim.x * 8) {
        float v[8];
        Vec8<T>::load(zr + i, v);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const float p2 = v[j] * v[j];
            s2 += p2;
            s4 = fmaf(p2, p2, s4);
            s6 = fmaf(p2 * p2, p2, s6);
        }
    }
    const float n = (float)n_mean;     // columns beyond n_mean are padding (zeros): they add nothing to the sums
    const float r1 = a * rsqrtf(block_sum(s2, scratch) / n + eps);
    const float r2 = b * rsqrtf(block_sum(s4, scratch) / n + eps);
    const float r3 = c * rsqrtf(block_sum(s6, scratch) / n + eps);
    for (int i = threadIdx.x * 8; i < inter; i += blockDim.x * 8) {
        float v[8], y[8];
        Vec8<T>::load(zr + i, v);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const float p2 = v[j] * v[j];
            y[j] = fmaf(r1, v[j], fmaf(r2, p2, fmaf(r3, p2 * v[j], e)));
        }
        Vec8<T>::store(o + i, y);
    }
}

cudaError_t launch_polynorm(int dtype, const void* z, const float* coef, float eps, void* out, int n_tokens, int inter,
                            int n_mean, cudaStream_t stream) {
    if (n_tokens == 0) return cudaSuccess;
    if (inter % 8) return cudaErrorInvalidValue;
    const int threads = min(512, max(32, ((inter / 8 + 31) / 32) * 32));
    if (dtype == kBF16)
        return launch(polynorm_kernel<__nv_bfloat16>, n_tokens, threads, 0, stream, (const __nv_bfloat16*)z, coef, eps, (__nv_bfloat16*)out, inter, n_mean);
    return launch(polynorm_kernel<float>, n_tokens, threads, 0, stream, (const float*)z, coef, eps, (float*)out, inter, n_mean);
}

// ------------------------------------------------------------------------- scaled copy into a range of columns

template <typename T>
__global__ void scale_into_kernel(const T* __restrict__ src, T* __restrict__ dst, long long total, int n, int dst_stride, int dst_col,
                                  float scale) {
    pdl_launch();
    pdl_wait();
    for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += (long long)gridDim.x * blockDim.x) {
        const long long t = e / n;
        const int i = (int)(e % n);
        dst[t * dst_stride + dst_col + i] = from_float<T>(to_float(src[e]) * scale);
    }
}

cudaError_t launch_scale_into(int dtype, const void* src, void* dst, int n_tokens, int n, int dst_stride, int dst_col, float scale,
                              cudaStream_t stream) {
    const long long total = (long long)n_tokens * n;
    if (total == 0) return cudaSuccess;
    const int blocks = (int)min((total + 255) / 256, (long long)148 * 16);
    if (dtype == kBF16)
        return launch(scale_into_kernel<__nv_bfloat16>, blocks, 256, 0, stream, (const __nv_bfloat16*)src, (__nv_bfloat16*)dst, total, n, dst_stride, dst_col, scale);
    return launch(scale_into_kernel<float>, blocks, 256, 0, stream, (const float*)src, (float*)dst, total, n, dst_stride, dst_col, scale);
}

template <typename T>
__global__ void gate_into_kernel(const T* __restrict__ src, const T* __restrict__ y, int y_stride, int gate_col, int mode,
                                 T* __restrict__ dst, long long total, int heads, int v_dim, int dst_stride, int dst_col, float scale) {
    pdl_launch();
    pdl_wait();
    const int n = heads * v_dim;
    for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += (long long)gridDim.x * blockDim.x) {
        const long long t = e / n;
        const int i = (int)(e % n);
        float v = to_float(src[e]) * scale;
        if (mode != 0) v *= 1.f / (1.f + expf(-to_float(y[t * y_stride + gate_col + (mode == 1 ? i / v_dim : i)])));
        dst[t * dst_stride + dst_col + i] = from_float<T>(v);
    }
}

cudaError_t launch_gate_into(int dtype, const void* src, const void* y, int y_stride, int gate_col, int mode, void* dst, int n_tokens,
                             int heads, int v_dim, int dst_stride, int dst_col, float scale, cudaStream_t stream) {
    const long long total = (long long)n_tokens * heads * v_dim;
    if (total == 0) return cudaSuccess;
    const int blocks = (int)min((total + 255) / 256, (long long)148 * 16);
    if (dtype == kBF16)
        return launch(gate_into_kernel<__nv_bfloat16>, blocks, 256, 0, stream, (const __nv_bfloat16*)src, (const __nv_bfloat16*)y, y_stride,
                      gate_col, mode, (__nv_bfloat16*)dst, total, heads, v_dim, dst_stride, dst_col, scale);
    return launch(gate_into_kernel<float>, blocks, 256, 0, stream, (const float*)src, (const float*)y, y_stride, gate_col, mode, (float*)dst,
                  total, heads, v_dim, dst_stride, dst_col, scale);
}

// ------------------------------------------------------------------------- silu * up

template <typename T>
__global__ void silu_mul_kernel(const T* __restrict__ gu, T* __restrict__ out, int n_tokens, int inter, int interleave) {
    pdl_launch();
    pdl_wait();
    const int per_row = inter / 8;
    const size_t total = (size_t)n_tokens * per_row;
    for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += (size_t)gridDim.x * blockDim.x) {
        const int t = (int)(e / per_row);
        const int i = (int)(e % per_row) * 8;
        float g[8], u[8], y[8];
        const T* row = gu + (size_t)t * 2 * inter;
        Vec8<T>::load(row + (interleave ? 2 * i : i), g);
        Vec8<T>::load(row + (interleave ? 2 * i + 8 : inter + i), u);
#pragma unroll
        for (int j = 0; j < 8; ++j) y[j] = g[j] / (1.f + expf(-g[j])) * u[j];
        Vec8<T>::store(out + (size_t)t * inter + i, y);
    }
}

cudaError_t launch_silu_mul(int dtype, const void* gu, void* out, int n_tokens, int inter, int interleave,
                            cudaStream_t stream) {
    if (interleave != 0 && interleave != 8) return cudaErrorInvalidValue;
    const size_t total = (size_t)n_tokens * (inter / 8);
    if (total == 0) return cudaSuccess;
    const int threads = 256;
    const int blocks = (int)min((size_t)148 * 16, (total + threads - 1) / threads);
    if (dtype == kBF16)
        return launch(silu_mul_kernel<__nv_bfloat16>, blocks, threads, 0, stream, (const __nv_bfloat16*)gu, (__nv_bfloat16*)out, n_tokens, inter, interleave);
    return launch(silu_mul_kernel<float>, blocks, threads, 0, stream, (const float*)gu, (float*)out, n_tokens, inter, interleave);
}

// ------------------------------------------------------------------------- rotation + cache store

// One block a token.  The angle's cos and sin come from a table of float pairs built on the
// host as vt-transformer builds its own (v1/tensortype/common.cpp:6-24); the rotation is done
// in 32-bit with one rounding.  Keys are rotated on their way into the page, values are copied.
template <typename T>
__global__ void rope_store_kernel(T* __restrict__ qkv, const int* __restrict__ positions,
                                  const float2* __restrict__ cos_sin, int max_pos, T* __restrict__ k_cache,
                                  T* __restrict__ v_cache, const int* __restrict__ token_seq,
                                  const int* __restrict__ block_table, int table_stride, int n_seqs, int n_pages,
                                  int heads, int kv_heads, int head_dim, int page_size, int rotate, int store,
                                  int* status) {
    // Positions, sequences and block tables are the step's own inputs, there before its first kernel starts: they are
    // read while the kernel before this one may still run; qkv, which that kernel writes, waits.  (Every thread
    // waits before it leaves: a kernel all of whose blocks left early would be done before the one before it.)
    pdl_launch();
    const int t = blockIdx.x;
    const int seq = token_seq[t];
    const bool seq_ok = seq >= 0 && seq < n_seqs;
    const int pos = seq_ok ? positions[t] : 0;
    const bool pos_ok = pos >= 0 && (!rotate || pos < max_pos);
    const int page = (store && seq_ok && pos_ok) ? block_table[(size_t)seq * table_stride + pos / page_size] : 0;
    pdl_wait();
    if (seq < 0) return;  // padding
    if (!seq_ok) {
        if (threadIdx.x == 0) set_status(status, kStatusBadSequence, seq);
        return;
    }
    if (!pos_ok) {
        if (threadIdx.x == 0) set_status(status, kStatusBadPosition, pos);
        return;
    }
    const int half = head_dim / 2;
    const int q_dim = heads * head_dim, kv_dim = kv_heads * head_dim;
    T* row = qkv + (size_t)t * (q_dim + 2 * kv_dim);
    const float2* cs = cos_sin + (size_t)pos * half;

    size_t page_base = 0;
    int slot = 0;
    if (store) {
        if (page < 0 || page >= n_pages) {
            if (threadIdx.x == 0) set_status(status, kStatusBadPage, page);
            store = 0;
        }
        page_base = (size_t)page * kv_heads * page_size * head_dim;
        slot = pos % page_size;
    }

    // eight pairs (i, i + half) at a time: 16- or 32-byte loads and stores (head_dim is a multiple of 16)
    auto rotate8 = [&](const T* src, T* dst, int i) {
        float a[8], b[8];
        Vec8<T>::load(src + i, a);
        Vec8<T>::load(src + i + half, b);
        if (rotate) {
            float c[16];
            Vec8<float>::load(reinterpret_cast<const float*>(cs + i), *reinterpret_cast<float(*)[8]>(c));
            Vec8<float>::load(reinterpret_cast<const float*>(cs + i) + 8, *reinterpret_cast<float(*)[8]>(c + 8));
            float ra[8], rb[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                ra[j] = a[j] * c[2 * j] - b[j] * c[2 * j + 1];
                rb[j] = b[j] * c[2 * j] + a[j] * c[2 * j + 1];
            }
            Vec8<T>::store(dst + i, ra);
            Vec8<T>::store(dst + i + half, rb);
        } else {
            Vec8<T>::store(dst + i, a);
            Vec8<T>::store(dst + i + half, b);
        }
    };
    const int half8 = half / 8;
    // queries: rotate in place
    if (rotate) {
        for (int e = threadIdx.x; e < heads * half8; e += blockDim.x) {
            T* p = row + (e / half8) * head_dim;
            rotate8(p, p, (e % half8) * 8);
        }
    }
    if (!store) return;
    // keys: rotate into the page
    for (int e = threadIdx.x; e < kv_heads * half8; e += blockDim.x) {
        const int h = e / half8;
        rotate8(row + q_dim + h * head_dim, k_cache + page_base + ((size_t)h * page_size + slot) * head_dim, (e % half8) * 8);
    }
    // values: copy into the page
    for (int e = threadIdx.x; e < kv_dim / 8; e += blockDim.x) {
        const int h = (e * 8) / head_dim, i = (e * 8) % head_dim;
        float v[8];
        Vec8<T>::load(row + q_dim + kv_dim + e * 8, v);
        Vec8<T>::store(v_cache + page_base + ((size_t)h * page_size + slot) * head_dim + i, v);
    }
}

cudaError_t launch_rope_store(int dtype, void* qkv, const int* positions, const float2* cos_sin, int max_pos,
                              void* k_cache, void* v_cache, const int* token_seq, const int* block_table,
                              int table_stride, int n_seqs, int n_pages, int n_tokens, int heads, int kv_heads,
                              int head_dim, int page_size, int rotate, int store, int* status, cudaStream_t stream) {
    if (n_tokens == 0) return cudaSuccess;
    if (head_dim % 16 != 0) return cudaErrorInvalidValue;       // eight pairs (i, i + head_dim / 2) a thread
    const int work = max(heads * head_dim / 16, kv_heads * head_dim / 8);
    const int threads = min(512, max(32, ((work + 31) / 32) * 32));
    if (dtype == kBF16)
        return launch(rope_store_kernel<__nv_bfloat16>, n_tokens, threads, 0, stream,
            (__nv_bfloat16*)qkv, positions, cos_sin, max_pos, (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache, token_seq,
            block_table, table_stride, n_seqs, n_pages, heads, kv_heads, head_dim, page_size, rotate, store, status);
    return launch(rope_store_kernel<float>, n_tokens, threads, 0, stream,
            (float*)qkv, positions, cos_sin, max_pos, (float*)k_cache, (float*)v_cache, token_seq, block_table,
            table_stride, n_seqs, n_pages, heads, kv_heads, head_dim, page_size, rotate, store, status);
}

}  // namespace vtb
