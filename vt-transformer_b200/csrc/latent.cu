// Kernels of layers that keep a narrow latent for each token instead of keys and values, and of what stands around
// them: the token shift, the norms of the two latents with the rotation of the shared key part and the store into the
// page, the products of each head with a matrix of its own (queries into the latent's space, the latent's result into
// the head's values), and two activations of feed-forwards.
//
// Latent attention in the absorbed form.  A token keeps c (the normed latent, `kv_rank` numbers) and one rotated key
// part r (`rot_dim` numbers) shared by all heads, side by side in one row of a page.  A head's key is [U_h c | r] and
// its value V_h c, so with q = [q_u | q_r]:  q . k = (U_h^T q_u) . c + q_r . r,  and  sum_j p_j V_h c_j = V_h (sum_j p_j c_j).
// The queries are therefore taken into the latent's space once a token (`head_matmul` with U_h, mode 1 also rotates
// q_r), the attention runs over the pages' rows as they lie (every head reads the same keys; a value is the first
// kv_rank numbers of its key's row), and the result is taken through V_h (`head_matmul` again, with the output gate).
#include "attention_mma.cuh"
#include "common.cuh"
#include "kernels.h"
#include "launch.cuh"

namespace vtb {

// ------------------------------------------------------------------------- token shift

// One block a token: out[t] = x[t] + (x[t - 1] - x[t]) * mu, where the token before a sequence's first token of this
// step is the row the sequence's state holds (zeros at its start).  The block of a sequence's first token of the step
// also leaves the sequence's last row of the step in the state: no other block touches that row of the state.
template <typename T>
__global__ void token_shift_kernel(const float* __restrict__ x, const float* __restrict__ mu, float* __restrict__ state,
                                   int state_rows, const int* __restrict__ cu_q, const int* __restrict__ rows,
                                   const int* __restrict__ token_seq, int n_seqs, T* __restrict__ out, int width, int* status) {
    pdl_launch();
    const int t = blockIdx.x;
    const int seq = token_seq[t];
    const bool ok = seq >= 0 && seq < n_seqs;
    const int first = ok ? cu_q[seq] : 0, last = ok ? cu_q[seq + 1] - 1 : 0, row = ok ? rows[seq] : 0;
    pdl_wait();
    T* o = out + (size_t)t * width;
    if (!ok) {
        if (seq >= n_seqs && threadIdx.x == 0) set_status(status, kStatusBadSequence, seq);
        for (int i = threadIdx.x; i < width; i += blockDim.x) o[i] = from_float<T>(0.f);      // padding
        return;
    }
    if (row < 0 || row >= state_rows) {
        if (threadIdx.x == 0) set_status(status, kStatusBadRow, row);
        return;
    }
    const float* xr = x + (size_t)t * width;
    float* sr = state + (size_t)row * width;
    const float* before = t == first ? sr : xr - width;
    const float* carry = x + (size_t)last * width;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        const float v = xr[i];
        o[i] = from_float<T>(fmaf(before[i] - v, mu[i], v));
        if (t == first) sr[i] = carry[i];           // read above by this thread, written by no other
    }
}

cudaError_t launch_token_shift(int out_dtype, const float* x, const float* mu, float* state, int state_rows, const int* cu_q,
                               const int* rows, const int* token_seq, int n_seqs, void* out, int n_tokens, int width, int* status,
                               cudaStream_t stream) {
    if (n_tokens == 0) return cudaSuccess;
    const int threads = min(512, max(32, ((width + 31) / 32) * 32));
    if (out_dtype == kBF16)
        return launch(token_shift_kernel<__nv_bfloat16>, n_tokens, threads, 0, stream, x, mu, state, state_rows, cu_q, rows, token_seq,
                      n_seqs, (__nv_bfloat16*)out, width, status);
    return launch(token_shift_kernel<float>, n_tokens, threads, 0, stream, x, mu, state, state_rows, cu_q, rows, token_seq, n_seqs,
                  (float*)out, width, status);
}

// ------------------------------------------------------------------------- the two latents of a token

// Pair i of a rotated vector, dimensions (2i, 2i + 1): (u, v) -> (u c - v s, v c + u s) with the angle pos * freq[i] formed
// as a 32-bit product and c, s multiplied by `mult`.
__device__ __forceinline__ void turn_pair(float u, float v, int pos, float f, float mult, float& a, float& b) {
    float sn, cs;
    sincosf((float)pos * f, &sn, &cs);
    sn *= mult;
    cs *= mult;
    a = u * cs - v * sn;
    b = v * cs + u * sn;
}

// One block a token.  y holds the results of the token's down projections: the queries' latent [q_rank] at q_col, and
// [kv_rank + rot_dim] at kv_col.  The queries' latent is divided by its root mean square, multiplied by q_weight and
// written to cq [tokens, cq_stride] (columns beyond q_rank are left).  The first kv_rank numbers at kv_col are normed
// the same way with k_weight, the last rot_dim are rotated by the token's position (the first 2 * half of them; not
// normed), and both go into the token's row of the page [pages, 1, page_size, kv_rank + rot_dim] if `store`.
template <typename T>
__global__ void latent_prepare_kernel(const T* __restrict__ y, int stride, int q_col, int q_rank, int kv_col, int kv_rank, int rot_dim,
                                      const float* __restrict__ q_weight, const float* __restrict__ k_weight, float eps,
                                      const float* __restrict__ freq, int half, float mult, const int* __restrict__ positions,
                                      const int* __restrict__ token_seq, const int* __restrict__ block_table, int table_stride,
                                      int n_seqs, int n_pages, int page_size, T* __restrict__ cq, int cq_stride, T* __restrict__ pages,
                                      int store, int* status) {
    __shared__ float scratch[32];
    pdl_launch();
    const int t = blockIdx.x;
    const int seq = token_seq[t];
    const bool seq_ok = seq >= 0 && seq < n_seqs;
    const int pos = seq_ok ? positions[t] : 0;
    const int page = (store && seq_ok && pos >= 0) ? block_table[(size_t)seq * table_stride + pos / page_size] : 0;
    pdl_wait();
    if (seq < 0) return;        // padding
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
    const T* row = y + (size_t)t * stride;
    // the queries' latent
    float ss = 0.f;
    for (int i = threadIdx.x; i < q_rank; i += blockDim.x) {
        const float v = to_float(row[q_col + i]);
        ss = fmaf(v, v, ss);
    }
    const float rq = rsqrtf(block_sum(ss, scratch) / (float)q_rank + eps);
    for (int i = threadIdx.x; i < q_rank; i += blockDim.x)
        cq[(size_t)t * cq_stride + i] = from_float<T>(to_float(row[q_col + i]) * rq * q_weight[i]);
    if (!store) return;
    // the keys' and values' latent, and the shared rotated key part
    ss = 0.f;
    for (int i = threadIdx.x; i < kv_rank; i += blockDim.x) {
        const float v = to_float(row[kv_col + i]);
        ss = fmaf(v, v, ss);
    }
    const float rk = rsqrtf(block_sum(ss, scratch) / (float)kv_rank + eps);
    T* dst = pages + ((size_t)page * page_size + pos % page_size) * (kv_rank + rot_dim);
    for (int i = threadIdx.x; i < kv_rank; i += blockDim.x) dst[i] = from_float<T>(to_float(row[kv_col + i]) * rk * k_weight[i]);
    const T* kr = row + kv_col + kv_rank;
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        float a, b;
        turn_pair(to_float(kr[2 * i]), to_float(kr[2 * i + 1]), pos, freq[i], mult, a, b);
        dst[kv_rank + 2 * i] = from_float<T>(a);
        dst[kv_rank + 2 * i + 1] = from_float<T>(b);
    }
    for (int i = 2 * half + threadIdx.x; i < rot_dim; i += blockDim.x) dst[kv_rank + i] = kr[i];
}

cudaError_t launch_latent_prepare(int dtype, const void* y, int stride, int q_col, int q_rank, int kv_col, int kv_rank, int rot_dim,
                                  const float* q_weight, const float* k_weight, float eps, const float* freq, int half, float mult,
                                  const int* positions, const int* token_seq, const int* block_table, int table_stride, int n_seqs,
                                  int n_pages, int page_size, void* cq, int cq_stride, void* pages, int store, int n_tokens, int* status,
                                  cudaStream_t stream) {
    if (n_tokens == 0) return cudaSuccess;
    if (2 * half > rot_dim) return cudaErrorInvalidValue;
    const int widest = max(q_rank, kv_rank);
    const int threads = min(512, max(32, ((widest + 31) / 32) * 32));
    if (dtype == kBF16)
        return launch(latent_prepare_kernel<__nv_bfloat16>, n_tokens, threads, 0, stream, (const __nv_bfloat16*)y, stride, q_col, q_rank,
                      kv_col, kv_rank, rot_dim, q_weight, k_weight, eps, freq, half, mult, positions, token_seq, block_table, table_stride,
                      n_seqs, n_pages, page_size, (__nv_bfloat16*)cq, cq_stride, (__nv_bfloat16*)pages, store, status);
    return launch(latent_prepare_kernel<float>, n_tokens, threads, 0, stream, (const float*)y, stride, q_col, q_rank, kv_col, kv_rank,
                  rot_dim, q_weight, k_weight, eps, freq, half, mult, positions, token_seq, block_table, table_stride, n_seqs, n_pages,
                  page_size, (float*)cq, cq_stride, (float*)pages, store, status);
}

// ------------------------------------------------------------------------- a product of each head with its own matrix

namespace {
constexpr int kHeadTokens = 8;       // tokens of a tile
constexpr int kHeadCols = 128;       // output columns of a tile, one a thread
}

// out[t, out_col + h * out_head + j] = sum_i x[t, x_col + h * x_head + i] * m[h, i, j]  for i < inner, j < outer, in 32-bit in
// the order of i (whatever else the step holds).  A block: 8 tokens, one head, 128 columns j; the tokens' inputs lie in
// shared memory ([i][token], so that a thread reads 8 tokens' values with two loads), a thread walks its column of m.
// mode 1 (queries into the latent's space): the `tail` numbers behind a head's `inner` inputs are its rotated part; they
// are turned by the token's position (pairs (2i, 2i + 1), the first 2 * half of them) and copied behind the head's
// `outer` outputs.  mode 2 (the latent's result into the head's values): the output is multiplied by
// sigmoid(gate[t, gate_col + h * outer + j]) where a gate is given.
template <typename T, typename TM>
__global__ void __launch_bounds__(kHeadCols)
head_matmul_kernel(const T* __restrict__ x, int x_stride, int x_col, int x_head, const TM* __restrict__ m, int inner, int outer,
                   T* __restrict__ out, int out_stride, int out_col, int out_head, int n_tokens, int mode, int tail,
                   const float* __restrict__ freq, int half, float mult, const int* __restrict__ positions,
                   const int* __restrict__ token_seq, const T* __restrict__ gate, int gate_stride, int gate_col) {
    extern __shared__ __align__(16) float xs[];            // [inner][8]
    pdl_launch();
    pdl_wait();
    const int t0 = blockIdx.x * kHeadTokens, h = blockIdx.y;
    const int j = blockIdx.z * kHeadCols + threadIdx.x;
    const int n = min(kHeadTokens, n_tokens - t0);
    for (int e = threadIdx.x; e < inner * kHeadTokens; e += kHeadCols) {
        const int tk = e / inner, i = e % inner;
        xs[i * kHeadTokens + tk] = tk < n ? to_float(x[(size_t)(t0 + tk) * x_stride + x_col + h * x_head + i]) : 0.f;
    }
    __syncthreads();
    float acc[kHeadTokens];
#pragma unroll
    for (int tk = 0; tk < kHeadTokens; ++tk) acc[tk] = 0.f;
    if (j < outer) {
        const TM* mp = m + (size_t)h * inner * outer + j;
#pragma unroll 4
        for (int i = 0; i < inner; ++i) {
            const float w = to_float(mp[(size_t)i * outer]);
            const float4 a = *reinterpret_cast<const float4*>(xs + i * kHeadTokens);
            const float4 b = *reinterpret_cast<const float4*>(xs + i * kHeadTokens + 4);
            acc[0] = fmaf(a.x, w, acc[0]); acc[1] = fmaf(a.y, w, acc[1]); acc[2] = fmaf(a.z, w, acc[2]); acc[3] = fmaf(a.w, w, acc[3]);
            acc[4] = fmaf(b.x, w, acc[4]); acc[5] = fmaf(b.y, w, acc[5]); acc[6] = fmaf(b.z, w, acc[6]); acc[7] = fmaf(b.w, w, acc[7]);
        }
#pragma unroll
        for (int tk = 0; tk < kHeadTokens; ++tk) {
            if (tk >= n) break;
            float v = acc[tk];
            if (mode == 2 && gate != nullptr) {
                const float z = to_float(gate[(size_t)(t0 + tk) * gate_stride + gate_col + h * outer + j]);
                v *= 1.f / (1.f + expf(-z));
            }
            out[(size_t)(t0 + tk) * out_stride + out_col + h * out_head + j] = from_float<T>(v);
        }
    }
    if (mode != 1 || blockIdx.z != 0) return;
    // the head's rotated part, behind its outputs
    for (int e = threadIdx.x; e < n * tail; e += kHeadCols) {
        const int tk = e / tail, i = e % tail, t = t0 + tk;
        const T* src = x + (size_t)t * x_stride + x_col + h * x_head + inner;
        float v = to_float(src[i]);
        if (i < 2 * half && token_seq[t] >= 0) {
            float a, b;
            const int pair = i >> 1;
            turn_pair(to_float(src[2 * pair]), to_float(src[2 * pair + 1]), positions[t], freq[pair], mult, a, b);
            v = (i & 1) ? b : a;
        }
        out[(size_t)t * out_stride + out_col + h * out_head + outer + i] = from_float<T>(v);
    }
}

// The same product on the tensor cores (bfloat16, 32-bit sums, one rounding), for steps with many tokens: a CTA forms 64
// tokens x 128 outputs of one head, its four warps 16 tokens each; x and M_h come in slices of 32 inner numbers through a
// two-stage cp.async pipeline (mma.sync m16n8k16; M_h's slice [inner][outer] is read transposed by ldmatrix).
constexpr int kHmRows = 64, kHmCols = 128, kHmInner = 32;

__global__ void __launch_bounds__(128)
head_matmul_mma_kernel(const __nv_bfloat16* __restrict__ x, int x_stride, int x_col, int x_head, const __nv_bfloat16* __restrict__ m,
                       int inner, int outer, __nv_bfloat16* __restrict__ out, int out_stride, int out_col, int out_head, int n_tokens,
                       int mode, int tail, const float* __restrict__ freq, int half, float mult, const int* __restrict__ positions,
                       const int* __restrict__ token_seq, const __nv_bfloat16* __restrict__ gate, int gate_stride, int gate_col) {
    constexpr int LA = kHmInner + 8, LB = kHmCols + 8;
    __shared__ __align__(16) __nv_bfloat16 as[2][kHmRows][LA];
    __shared__ __align__(16) __nv_bfloat16 bs[2][kHmInner][LB];
    pdl_launch();
    pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, gq = lane >> 2, tq = lane & 3;
    const int t0 = blockIdx.x * kHmRows, h = blockIdx.y, n0 = blockIdx.z * kHmCols;
    const int n = min(kHmRows, n_tokens - t0);
    const __nv_bfloat16* xh = x + (size_t)t0 * x_stride + x_col + (size_t)h * x_head;
    const __nv_bfloat16* mh = m + (size_t)h * inner * outer + n0;
    auto load_slice = [&](int k0, int stage) {
        for (int c = threadIdx.x; c < kHmRows * (kHmInner / 8); c += 128) {
            const int r = c / (kHmInner / 8), piece = c % (kHmInner / 8);
            const bool ok = r < n && k0 + piece * 8 < inner;
            cp_async16(&as[stage][r][piece * 8], xh + (ok ? (size_t)r * x_stride + k0 + piece * 8 : 0), ok);
        }
        for (int c = threadIdx.x; c < kHmInner * (kHmCols / 8); c += 128) {
            const int r = c / (kHmCols / 8), piece = c % (kHmCols / 8);
            const bool ok = k0 + r < inner && n0 + piece * 8 < outer;
            cp_async16(&bs[stage][r][piece * 8], mh + (ok ? (size_t)(k0 + r) * outer + piece * 8 : 0), ok);
        }
    };
    float acc[kHmCols / 8][4];
#pragma unroll
    for (int i = 0; i < kHmCols / 8; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;
    const int slices = (inner + kHmInner - 1) / kHmInner;
    load_slice(0, 0);
    cp_async_commit();
    for (int sl = 0; sl < slices; ++sl) {
        const int stage = sl & 1;
        if (sl + 1 < slices) load_slice((sl + 1) * kHmInner, stage ^ 1);
        cp_async_commit();
        cp_async_wait<1>();
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < kHmInner / 16; ++kk) {
            uint32_t af[4];
            ldmatrix_x4(af, &as[stage][warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8][kk * 16 + (lane >> 4) * 8]);
            const int mat = lane >> 3, r = lane & 7;
#pragma unroll
            for (int dn = 0; dn < kHmCols / 16; ++dn) {
                if (n0 + dn * 16 < outer) {
                    uint32_t bf[4];
                    ldmatrix_x4_trans(bf, &bs[stage][kk * 16 + (mat & 1) * 8 + r][dn * 16 + (mat >> 1) * 8]);
                    mma_bf16(acc[2 * dn], af, bf[0], bf[1]);
                    mma_bf16(acc[2 * dn + 1], af, bf[2], bf[3]);
                }
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int tk = warp * 16 + gq + 8 * i;
        if (tk >= n) continue;
        __nv_bfloat16* op = out + (size_t)(t0 + tk) * out_stride + out_col + (size_t)h * out_head;
        const __nv_bfloat16* gp = (mode == 2 && gate != nullptr) ? gate + (size_t)(t0 + tk) * gate_stride + gate_col + (size_t)h * outer : nullptr;
#pragma unroll
        for (int nt = 0; nt < kHmCols / 8; ++nt) {
            const int j = n0 + nt * 8 + 2 * tq;
            if (j >= outer) continue;
            float v0 = acc[nt][2 * i], v1 = acc[nt][2 * i + 1];
            if (gp) {
                v0 *= 1.f / (1.f + expf(-__bfloat162float(gp[j])));
                v1 *= 1.f / (1.f + expf(-__bfloat162float(gp[j + 1])));
            }
            *reinterpret_cast<uint32_t*>(op + j) = pack_bf16(v0, v1);
        }
    }
    if (mode != 1 || blockIdx.z != 0) return;
    // the head's rotated part, behind its outputs
    for (int e = threadIdx.x; e < n * tail; e += 128) {
        const int tk = e / tail, i = e % tail, t = t0 + tk;
        const __nv_bfloat16* src = x + (size_t)t * x_stride + x_col + h * x_head + inner;
        float v = __bfloat162float(src[i]);
        if (i < 2 * half && token_seq[t] >= 0) {
            float a, b;
            const int pair = i >> 1;
            turn_pair(__bfloat162float(src[2 * pair]), __bfloat162float(src[2 * pair + 1]), positions[t], freq[pair], mult, a, b);
            v = (i & 1) ? b : a;
        }
        out[(size_t)t * out_stride + out_col + h * out_head + outer + i] = __float2bfloat16_rn(v);
    }
}

// from how many tokens on a step's products of the heads run on the tensor cores (below, M_h's bytes bound the time)
constexpr int kHmMinTokens = 32;

cudaError_t launch_head_matmul(int dtype, int m_dtype, const void* x, int x_stride, int x_col, int x_head, const void* m, int heads,
                               int inner, int outer, void* out, int out_stride, int out_col, int out_head, int n_tokens, int mode,
                               int tail, const float* freq, int half, float mult, const int* positions, const int* token_seq,
                               const void* gate, int gate_stride, int gate_col, cudaStream_t stream) {
    if (n_tokens == 0 || heads == 0) return cudaSuccess;
    if (2 * half > tail || (mode == 1 && half > 0 && (freq == nullptr || positions == nullptr || token_seq == nullptr)))
        return cudaErrorInvalidValue;
    if (dtype == kBF16 && m_dtype == kBF16 && n_tokens >= kHmMinTokens && inner % 8 == 0 && outer % 8 == 0 && x_stride % 8 == 0 &&
        x_col % 8 == 0 && x_head % 8 == 0 && out_stride % 2 == 0 && out_col % 2 == 0 && out_head % 2 == 0 &&
        ((uintptr_t)x & 15) == 0 && ((uintptr_t)m & 15) == 0 && ((uintptr_t)out & 3) == 0) {
        const dim3 grid_mma((n_tokens + kHmRows - 1) / kHmRows, heads, (outer + kHmCols - 1) / kHmCols);
        return launch(head_matmul_mma_kernel, grid_mma, 128, 0, stream, (const __nv_bfloat16*)x, x_stride, x_col, x_head,
                      (const __nv_bfloat16*)m, inner, outer, (__nv_bfloat16*)out, out_stride, out_col, out_head, n_tokens, mode, tail, freq,
                      half, mult, positions, token_seq, (const __nv_bfloat16*)gate, gate_stride, gate_col);
    }
    const size_t bytes = (size_t)inner * kHeadTokens * sizeof(float);
    if (bytes > 48 * 1024) return cudaErrorInvalidValue;                     // inner sizes up to 1,536
    const dim3 grid((n_tokens + kHeadTokens - 1) / kHeadTokens, heads, (outer + kHeadCols - 1) / kHeadCols);
    if (dtype == kBF16 && m_dtype == kBF16)
        return launch(head_matmul_kernel<__nv_bfloat16, __nv_bfloat16>, grid, kHeadCols, bytes, stream, (const __nv_bfloat16*)x, x_stride,
                      x_col, x_head, (const __nv_bfloat16*)m, inner, outer, (__nv_bfloat16*)out, out_stride, out_col, out_head, n_tokens,
                      mode, tail, freq, half, mult, positions, token_seq, (const __nv_bfloat16*)gate, gate_stride, gate_col);
    if (dtype == kBF16 && m_dtype == kF32)
        return launch(head_matmul_kernel<__nv_bfloat16, float>, grid, kHeadCols, bytes, stream, (const __nv_bfloat16*)x, x_stride, x_col,
                      x_head, (const float*)m, inner, outer, (__nv_bfloat16*)out, out_stride, out_col, out_head, n_tokens, mode, tail,
                      freq, half, mult, positions, token_seq, (const __nv_bfloat16*)gate, gate_stride, gate_col);
    if (dtype == kF32 && m_dtype == kF32)
        return launch(head_matmul_kernel<float, float>, grid, kHeadCols, bytes, stream, (const float*)x, x_stride, x_col, x_head,
                      (const float*)m, inner, outer, (float*)out, out_stride, out_col, out_head, n_tokens, mode, tail, freq, half, mult,
                      positions, token_seq, (const float*)gate, gate_stride, gate_col);
    return cudaErrorInvalidValue;
}

// ------------------------------------------------------------------------- activations of feed-forwards

// xIELU, element by element in 32-bit with one rounding: for z > 0  ap z^2 + z / 2;  for z <= 0  an (exp(z) - 1 - z) + z / 2.
// (ap = softplus(p) and an = 1/2 + softplus(q) of the layer's two numbers are formed when the weights are loaded.)
template <typename T>
__global__ void xielu_kernel(const T* __restrict__ z, T* __restrict__ out, long long n, float ap, float an) {
    pdl_launch();
    pdl_wait();
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        const float v = to_float(z[i]);
        out[i] = from_float<T>(v > 0.f ? fmaf(ap * v, v, 0.5f * v) : fmaf(an, expm1f(v) - v, 0.5f * v));
    }
}

cudaError_t launch_xielu(int dtype, const void* z, void* out, long long n, float ap, float an, cudaStream_t stream) {
    if (n == 0) return cudaSuccess;
    const int blocks = (int)min((n + 255) / 256, (long long)148 * 16);
    if (dtype == kBF16)
        return launch(xielu_kernel<__nv_bfloat16>, blocks, 256, 0, stream, (const __nv_bfloat16*)z, (__nv_bfloat16*)out, n, ap, an);
    return launch(xielu_kernel<float>, blocks, 256, 0, stream, (const float*)z, (float*)out, n, ap, an);
}

// The clamped gate: with g = min(gate, limit) and u = clamp(up, -limit, limit):  out = g * sigmoid(alpha * g) * (u + 1).
// gu [tokens, 2 * inter] holds gate and up side by side ([gate | up]) or, with `interleave` 8, alternating in runs of 8.
// Columns from `split` on (of out) take `limit2` (an expert of its own constants behind the others'); 32-bit, one rounding.
template <typename T>
__global__ void gate_clamp_kernel(const T* __restrict__ gu, T* __restrict__ out, int n_tokens, int inter, int interleave, float alpha,
                                  float limit, int split, float limit2) {
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
        const float lim = i >= split ? limit2 : limit;
#pragma unroll
        for (int j = 0; j < 8; ++j) y[j] = gate_clamp(g[j], u[j], alpha, lim);
        Vec8<T>::store(out + (size_t)t * inter + i, y);
    }
}

cudaError_t launch_gate_clamp(int dtype, const void* gu, void* out, int n_tokens, int inter, int interleave, float alpha, float limit,
                              int split, float limit2, cudaStream_t stream) {
    if ((interleave != 0 && interleave != 8) || inter % 8 || split % 8) return cudaErrorInvalidValue;
    const size_t total = (size_t)n_tokens * (inter / 8);
    if (total == 0) return cudaSuccess;
    const int blocks = (int)min((size_t)148 * 16, (total + 255) / 256);
    if (dtype == kBF16)
        return launch(gate_clamp_kernel<__nv_bfloat16>, blocks, 256, 0, stream, (const __nv_bfloat16*)gu, (__nv_bfloat16*)out, n_tokens,
                      inter, interleave, alpha, limit, split, limit2);
    return launch(gate_clamp_kernel<float>, blocks, 256, 0, stream, (const float*)gu, (float*)out, n_tokens, inter, interleave, alpha, limit,
                  split, limit2);
}

}  // namespace vtb
