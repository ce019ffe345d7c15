// Recurrences that carry a matrix for each (request, head) and scale it by one number a token: the delta rule with one
// decay a head (with short convolutions over time in front of q, k and v), and the matrix memory with exponential gates.
// Beside them the small kernels of a mixer whose branches' results are normed before they are added.
//
// For one head with state S [dim, v_dim] in 32-bit:
//   delta rule     S <- g_t S;  u = beta_t (v_t - S^T k_t);  S <- S + k_t u^T;            o_t = S^T q_t
//   matrix memory  m' = max(f_t + m, i_t);  S <- exp(f_t + m - m') S + exp(i_t - m') k_t v_t^T;  n likewise with k_t alone;
//                  o_t = S^T q_t / (max(|n . q_t|, exp(-m')) + eps)
// Column j of S depends on column j alone: a warp owns 32 columns of one (sequence, head), a thread keeps KD rows of its
// column in registers (8), and G = dim / 8 threads share a column (their partial sums meet in shared memory, in the
// order of g).  The step's tokens of the sequence are staged 16 at a time: the convolutions and their silu, the unit
// vectors, the gates, the running maximum and the normalizer are formed once for all columns, in 32-bit; then the
// warps walk the batch out of shared memory.  A decoded token is a walk of one token.  The order of every sum depends
// on the sizes alone, never on how the tokens were cut into steps.
#include "common.cuh"
#include "kernels.h"
#include "launch.cuh"

namespace vtb {

namespace {

constexpr int kCols = 32;        // columns of the state a warp owns
constexpr int kTokens = 16;      // tokens staged at once in steps of single tokens and short portions
constexpr int kWalkTokens = 32;  // ... and in long walks, where the staging's fixed waits weigh more
constexpr int kRows = 8;         // rows of its column that a thread keeps in registers
constexpr int kMaxThreads = 1024;
// Threads of a CTA in a step that is a long walk of few sequences: a head's column blocks then spread over several SMs
// (each forms the gates again); steps of single tokens keep as many of a head's columns in one CTA as fit.
constexpr int kWalkThreads = 512;

struct GatedArgs {
    const void* y;               // [tokens, stride]: the projections
    int stride;
    int q_col, k_col, v_col;
    int g1_col, g2_col;          // delta rule: beta's and the decay's inputs; matrix memory: the input and forget gates'
    const float* conv_q;         // delta rule: [channels, taps] each
    const float* conv_k;
    const float* conv_v;
    int taps;
    const float* p1;             // delta rule: a_log [heads]; matrix memory: the input gate's bias
    const float* p2;             // delta rule: dt_bias [heads]; matrix memory: the forget gate's bias
    float c1, c2, c3;            // delta rule: eps of the unit vectors, the scale of q; matrix memory: the gates' cap, the scale of q, eps of the denominator
    float* state;
    int state_rows;
    const float* tail;           // delta rule: [state_rows, taps - 1, tail_channels], or null
    int tail_channels;
    // matrix memory with a head's columns on several CTAs: n and m as they were before the step, [sequences, heads, dim + 1]
    // (the CTA of the first columns renews them in the state while others may not have read them yet); else null
    const float* snap;
    const int* cu_q;
    const int* rows;
    float* out;
    int heads, kv_heads, dim, v_dim, groups, col_blocks;
    int* status;
};

__device__ __forceinline__ float sigmoid_f(float z) { return 1.f / (1.f + expf(-z)); }
__device__ __forceinline__ float softplus_f(float z) { return z > 20.f ? z : log1pf(expf(z)); }
__device__ __forceinline__ float log_sigmoid_f(float z) { return z < 0.f ? z - log1pf(expf(z)) : -log1pf(expf(-z)); }

// MODE 0: the delta rule; 1: the matrix memory.  Block (32, G, CB): thread (c, g, cb) keeps rows [g KD, (g + 1) KD) of column
// blockIdx.z * CB * 32 + cb * 32 + c.
// WALK: the variant for long walks of few sequences, compiled for CTAs of 256 threads (and the registers they may have).
template <typename T, int KD, int MODE, bool WALK>
__global__ void __launch_bounds__(WALK ? kWalkThreads : kMaxThreads, 1)
gated_scan_kernel(const GatedArgs a) {
    extern __shared__ __align__(16) float smem[];
    pdl_launch();
    const int seq = blockIdx.x, h = blockIdx.y;
    const int c = threadIdx.x, g = threadIdx.y, cb = threadIdx.z;
    const int G = a.groups, CB = a.col_blocks;
    constexpr int TB = WALK ? kWalkTokens : kTokens;
    const int tid = (cb * G + g) * kCols + c, n_threads = kCols * G * CB;
    const int warp = tid >> 5, n_warps = n_threads >> 5;
    const int dim = a.dim, v_dim = a.v_dim;
    const int dim_p = G * KD, cols = CB * kCols;
    const int col0 = blockIdx.z * cols;
    const int j = col0 + cb * kCols + c;
    const bool col_ok = j < v_dim;
    const int taps = MODE == 0 ? a.taps : 1;
    const int kvh = h / (a.heads / a.kv_heads);
    const int per = 2 * dim_p + cols;                       // values of a token that the CTA reads: q, k and its columns of v
    float* qs = smem;                                       // [TB, dim_p]
    float* ks = qs + TB * dim_p;                            // [TB, dim_p]
    float* vs = ks + TB * dim_p;                            // [TB, cols]
    float* sc = vs + TB * cols;                             // [TB, 4]: the token's scalars
    float* red = sc + TB * 4;                               // [2, CB, G, 32]: where the groups of a column meet inside a token
    float* op = red + 2 * CB * G * kCols;                   // [TB, G, cols]: the groups' shares of the outputs
    float* extra = op + TB * G * cols;
    float* raw = extra;                                     // delta rule: [TB + taps - 1, per] inputs of the convolutions
    float* wc = raw + (TB + taps - 1) * per;                // delta rule: [taps, per] the convolutions' weights of these channels
    float* nq = extra;                                      // matrix memory: [TB, dim_p] products n_i q_i
    float* m_cur = extra + TB * dim_p;                      // matrix memory: the running maximum

    // channel `ch` of the CTA's values: which vector it belongs to, whether it exists, where it lies in y and in the kept inputs
    const int nqk = a.kv_heads * dim;
    auto channel = [&](int ch, int& y_col, int& t_col) -> bool {
        if (ch < 2 * dim_p) {
            const int which = ch < dim_p ? 0 : 1, i = ch - which * dim_p;
            if (i >= dim) return false;
            const int at = (MODE == 0 ? kvh : h) * dim + i;
            y_col = (which == 0 ? a.q_col : a.k_col) + at;
            t_col = which * nqk + at;
            return true;
        }
        const int cc = ch - 2 * dim_p;
        if (col0 + cc >= v_dim) return false;
        y_col = a.v_col + h * v_dim + col0 + cc;
        t_col = 2 * nqk + h * v_dim + col0 + cc;
        return true;
    };
    if (MODE == 0) {
        // the weights are written by no kernel of the step: they are read before the wait
        for (int e = tid; e < taps * per; e += n_threads) {
            const int tap = e / per, ch = e % per;
            int y_col = 0, t_col = 0;
            float w = 0.f;
            if (channel(ch, y_col, t_col)) {
                const float* base = t_col < nqk ? a.conv_q + (size_t)t_col * taps
                                    : (t_col < 2 * nqk ? a.conv_k + (size_t)(t_col - nqk) * taps : a.conv_v + (size_t)(t_col - 2 * nqk) * taps);
                w = base[tap];
            }
            wc[e] = w;
        }
    }
    pdl_wait();
    const int t0 = a.cu_q[seq], t1 = a.cu_q[seq + 1];
    if (t1 <= t0) return;                                   // a sequence without tokens in this step (padding): its state stays
    const int row = a.rows[seq];
    if (row < 0 || row >= a.state_rows) {
        if (tid == 0) set_status(a.status, kStatusBadRow, row);
        return;
    }
    const T* y = reinterpret_cast<const T*>(a.y);
    const int s_rows = MODE == 0 ? dim : dim + 1, s_cols = MODE == 0 ? v_dim : v_dim + 1;
    float* sp = a.state + ((size_t)row * a.heads + h) * s_rows * s_cols;
    float S[KD];
#pragma unroll
    for (int i = 0; i < KD; ++i) {
        const int r = g * KD + i;
        S[i] = (col_ok && r < dim) ? sp[(size_t)r * s_cols + j] : 0.f;
    }
    float n_i = 0.f;                                        // matrix memory: thread i < dim keeps n_i
    if (MODE == 1) {
        const float* before = a.snap != nullptr ? a.snap + ((size_t)seq * a.heads + h) * (dim + 1) : nullptr;
        if (tid < dim) n_i = before ? before[tid] : sp[(size_t)tid * s_cols + v_dim];
        if (tid == 0) *m_cur = before ? before[dim] : sp[(size_t)dim * s_cols];
    }
    int meet = 0;
    for (int tb0 = t0; tb0 < t1; tb0 += TB) {
        const int n = min(TB, t1 - tb0);
        __syncthreads();                                    // the batch before is done with
        if (MODE == 0) {
            // the convolutions' inputs of the batch and of the taps - 1 tokens before it: from y, or from the kept inputs
            for (int e = tid; e < (n + taps - 1) * per; e += n_threads) {
                const int r = e / per, ch = e % per;
                const int s = tb0 - (taps - 1) + r;
                int y_col = 0, t_col = 0;
                float v = 0.f;
                if (channel(ch, y_col, t_col)) {
                    if (s >= t0) v = to_float(y[(size_t)s * a.stride + y_col]);
                    else if (a.tail != nullptr) v = a.tail[((size_t)row * (taps - 1) + (taps - 1) - (t0 - s)) * a.tail_channels + t_col];
                }
                raw[e] = v;
            }
            for (int tb = tid; tb < n; tb += n_threads) {
                const T* yr = y + (size_t)(tb0 + tb) * a.stride;
                sc[tb * 4 + 0] = expf(-expf(a.p1[h]) * softplus_f(to_float(yr[a.g2_col + h]) + a.p2[h]));     // the decay
                sc[tb * 4 + 1] = sigmoid_f(to_float(yr[a.g1_col + h]));                                        // beta
            }
            __syncthreads();
            for (int e = tid; e < n * per; e += n_threads) {
                const int tb = e / per, ch = e % per;
                float z = 0.f;
                for (int tap = 0; tap < taps; ++tap) z = fmaf(wc[tap * per + ch], raw[(tb + tap) * per + ch], z);
                z = z / (1.f + expf(-z));
                if (ch < dim_p) qs[tb * dim_p + ch] = z;
                else if (ch < 2 * dim_p) ks[tb * dim_p + ch - dim_p] = z;
                else vs[tb * cols + ch - 2 * dim_p] = z;
            }
            __syncthreads();
            // unit q and k (q with its scale): a warp for each staged token
            for (int tb = warp; tb < n; tb += n_warps) {
                float sq = 0.f, sk = 0.f;
                for (int i = c; i < dim_p; i += 32) {
                    sq = fmaf(qs[tb * dim_p + i], qs[tb * dim_p + i], sq);
                    sk = fmaf(ks[tb * dim_p + i], ks[tb * dim_p + i], sk);
                }
                const float iq = a.c2 / sqrtf(warp_sum(sq) + a.c1), ik = 1.f / sqrtf(warp_sum(sk) + a.c1);
                for (int i = c; i < dim_p; i += 32) {
                    qs[tb * dim_p + i] *= iq;
                    ks[tb * dim_p + i] *= ik;
                }
            }
            __syncthreads();
        } else {
            for (int e = tid; e < n * per; e += n_threads) {
                const int tb = e / per, ch = e % per;
                int y_col = 0, t_col = 0;
                const float v = channel(ch, y_col, t_col) ? to_float(y[(size_t)(tb0 + tb) * a.stride + y_col]) : 0.f;
                if (ch < dim_p) qs[tb * dim_p + ch] = v * a.c2;
                else if (ch < 2 * dim_p) ks[tb * dim_p + ch - dim_p] = v;
                else vs[tb * cols + ch - 2 * dim_p] = v;
            }
            for (int tb = tid; tb < n; tb += n_threads) {
                const T* yr = y + (size_t)(tb0 + tb) * a.stride;
                const float cap = a.c1;
                sc[tb * 4 + 0] = cap * tanhf((to_float(yr[a.g1_col + h]) + a.p1[h]) / cap);                   // log of the input gate
                sc[tb * 4 + 1] = log_sigmoid_f(cap * tanhf((to_float(yr[a.g2_col + h]) + a.p2[h]) / cap));    // log of the forget gate
            }
            __syncthreads();
            if (tid == 0) {
                // the running maximum and the two factors of every token of the batch, one after the other
                float m = *m_cur;
                for (int tb = 0; tb < n; ++tb) {
                    const float ig = sc[tb * 4 + 0], fg = sc[tb * 4 + 1];
                    const float m_new = fmaxf(fg + m, ig);
                    sc[tb * 4 + 0] = expf(fg + m - m_new);
                    sc[tb * 4 + 1] = expf(ig - m_new);
                    sc[tb * 4 + 2] = expf(-m_new);
                    m = m_new;
                }
                *m_cur = m;
            }
            __syncthreads();
            if (tid < dim_p) {
                for (int tb = 0; tb < n; ++tb) {
                    n_i = fmaf(sc[tb * 4 + 0], n_i, sc[tb * 4 + 1] * ks[tb * dim_p + tid]);
                    nq[tb * dim_p + tid] = n_i * qs[tb * dim_p + tid];
                }
            }
            __syncthreads();
            for (int tb = warp; tb < n; tb += n_warps) {
                float s = 0.f;
                for (int i = c; i < dim_p; i += 32) s += nq[tb * dim_p + i];
                s = warp_sum(s);
                if (c == 0) sc[tb * 4 + 3] = fmaxf(fabsf(s), sc[tb * 4 + 2]) + a.c3;
            }
            __syncthreads();
        }
        for (int tb = 0; tb < n; ++tb) {
            const float v = vs[tb * cols + cb * kCols + c];
            const float4* q4 = reinterpret_cast<const float4*>(qs + tb * dim_p + g * KD);
            const float4* k4 = reinterpret_cast<const float4*>(ks + tb * dim_p + g * KD);
            const float s0 = sc[tb * 4 + 0], s1 = sc[tb * 4 + 1];
            float acc[4] = {0.f, 0.f, 0.f, 0.f};
            if (MODE == 0) {
                float part[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                for (int i = 0; i < KD / 4; ++i) {
                    const float4 k = k4[i];
                    S[4 * i + 0] *= s0; S[4 * i + 1] *= s0; S[4 * i + 2] *= s0; S[4 * i + 3] *= s0;
                    part[0] = fmaf(k.x, S[4 * i + 0], part[0]);
                    part[1] = fmaf(k.y, S[4 * i + 1], part[1]);
                    part[2] = fmaf(k.z, S[4 * i + 2], part[2]);
                    part[3] = fmaf(k.w, S[4 * i + 3], part[3]);
                }
                float ks_old = (part[0] + part[1]) + (part[2] + part[3]);
                if (G > 1) {
                    // S^T k of the decayed state is needed before the update: the G warps that share these columns meet
                    // (a barrier of their own; two buffers in turn, so one meeting a token is enough)
                    float* m = red + ((meet++ & 1) * CB + cb) * G * kCols;
                    m[g * kCols + c] = ks_old;
                    asm volatile("bar.sync %0, %1;" ::"r"(cb + 1), "r"(G * kCols) : "memory");
                    ks_old = 0.f;
                    for (int gg = 0; gg < G; ++gg) ks_old += m[gg * kCols + c];
                }
                const float u = s1 * (v - ks_old);
#pragma unroll
                for (int i = 0; i < KD / 4; ++i) {
                    const float4 q = q4[i], k = k4[i];
                    S[4 * i + 0] = fmaf(k.x, u, S[4 * i + 0]);
                    S[4 * i + 1] = fmaf(k.y, u, S[4 * i + 1]);
                    S[4 * i + 2] = fmaf(k.z, u, S[4 * i + 2]);
                    S[4 * i + 3] = fmaf(k.w, u, S[4 * i + 3]);
                    acc[0] = fmaf(S[4 * i + 0], q.x, acc[0]);
                    acc[1] = fmaf(S[4 * i + 1], q.y, acc[1]);
                    acc[2] = fmaf(S[4 * i + 2], q.z, acc[2]);
                    acc[3] = fmaf(S[4 * i + 3], q.w, acc[3]);
                }
            } else {
                const float bv = s1 * v;
#pragma unroll
                for (int i = 0; i < KD / 4; ++i) {
                    const float4 q = q4[i], k = k4[i];
                    S[4 * i + 0] = fmaf(s0, S[4 * i + 0], k.x * bv);
                    S[4 * i + 1] = fmaf(s0, S[4 * i + 1], k.y * bv);
                    S[4 * i + 2] = fmaf(s0, S[4 * i + 2], k.z * bv);
                    S[4 * i + 3] = fmaf(s0, S[4 * i + 3], k.w * bv);
                    acc[0] = fmaf(S[4 * i + 0], q.x, acc[0]);
                    acc[1] = fmaf(S[4 * i + 1], q.y, acc[1]);
                    acc[2] = fmaf(S[4 * i + 2], q.z, acc[2]);
                    acc[3] = fmaf(S[4 * i + 3], q.w, acc[3]);
                }
            }
            // this group's share of the token's output; the sum over the groups is formed once the batch is through
            op[(tb * G + g) * cols + cb * kCols + c] = (acc[0] + acc[1]) + (acc[2] + acc[3]);
        }
        __syncthreads();
        for (int e = tid; e < n * cols; e += n_threads) {
            const int tb = e / cols, cc = e % cols;
            if (col0 + cc >= v_dim) continue;
            float o = 0.f;
            for (int gg = 0; gg < G; ++gg) o += op[(tb * G + gg) * cols + cc];
            if (MODE == 1) o /= sc[tb * 4 + 3];
            a.out[(size_t)(tb0 + tb) * a.heads * v_dim + (size_t)h * v_dim + col0 + cc] = o;
        }
    }
#pragma unroll
    for (int i = 0; i < KD; ++i) {
        const int r = g * KD + i;
        if (col_ok && r < dim) sp[(size_t)r * s_cols + j] = S[i];
    }
    if (MODE == 1 && blockIdx.z == 0) {
        // (the last batch's barriers lie behind every write of m_cur)
        if (tid < dim) sp[(size_t)tid * s_cols + v_dim] = n_i;
        if (tid == 0) sp[(size_t)dim * s_cols] = *m_cur;
    }
}

// n and m of every (sequence, head) of the step as they are before it.
__global__ void memory_snapshot_kernel(const float* __restrict__ state, int state_rows, const int* __restrict__ cu_q,
                                       const int* __restrict__ rows, float* __restrict__ snap, int heads, int dim, int v_dim) {
    pdl_launch();
    pdl_wait();
    const int seq = blockIdx.x, h = blockIdx.y;
    if (cu_q[seq + 1] <= cu_q[seq]) return;
    const int row = rows[seq];
    if (row < 0 || row >= state_rows) return;               // the scan reports it
    const float* sp = state + ((size_t)row * heads + h) * (dim + 1) * (v_dim + 1);
    float* out = snap + ((size_t)seq * heads + h) * (dim + 1);
    for (int i = threadIdx.x; i <= dim; i += blockDim.x) out[i] = i < dim ? sp[(size_t)i * (v_dim + 1) + v_dim] : sp[(size_t)dim * (v_dim + 1)];
}

template <typename T, int KD, int MODE>
cudaError_t launch_gated_kd(const GatedArgs& a, int n_seqs, int most_threads, cudaStream_t stream) {
    GatedArgs args = a;
    const int G = (a.dim + KD - 1) / KD;
    const int limit = most_threads > 0 ? max(kCols * G, min(most_threads, kMaxThreads)) : kMaxThreads;
    // the matrix memory's normalizer wants a thread for every row of the head: at least dim_p threads
    int cb = max(1, min((a.v_dim + kCols - 1) / kCols, limit / (kCols * G)));
    cb = min(cb, 15);                                       // the groups' barriers are numbered 1 to 15
    if (cb > 15 || cb * kCols * G > kMaxThreads) return cudaErrorInvalidValue;
    args.groups = G;
    args.col_blocks = cb;
    const int dim_p = G * KD, cols = cb * kCols, per = 2 * dim_p + cols;
    const int taps = MODE == 0 ? a.taps : 1;
    const bool walk = most_threads > 0 && cb * kCols * G <= kWalkThreads;
    const int tb = walk ? kWalkTokens : kTokens;
    size_t floats = (size_t)2 * tb * dim_p + tb * cols + tb * 4 + 2 * cb * G * kCols + (size_t)tb * G * cols;
    floats += MODE == 0 ? (size_t)(tb + taps - 1) * per + (size_t)taps * per : (size_t)tb * dim_p + 4;
    const size_t bytes = floats * sizeof(float);
    if (bytes > 200 * 1024) return cudaErrorInvalidValue;
    auto kernel = walk ? gated_scan_kernel<T, KD, MODE, true> : gated_scan_kernel<T, KD, MODE, false>;
    static std::atomic<unsigned long long> done[2] = {{0}, {0}};
    if (cudaError_t e = allow_dynamic_smem(kernel, 200 * 1024, done[walk ? 1 : 0]); e != cudaSuccess) return e;
    const dim3 grid(n_seqs, a.heads, (a.v_dim + cols - 1) / cols), block(kCols, G, cb);
    if (MODE == 1) {
        if (grid.z > 1) {
            if (a.snap == nullptr) return cudaErrorInvalidValue;
            if (cudaError_t e = launch(memory_snapshot_kernel, dim3(n_seqs, a.heads), 128, 0, stream, a.state, a.state_rows, a.cu_q, a.rows,
                                       const_cast<float*>(a.snap), a.heads, a.dim, a.v_dim); e != cudaSuccess) return e;
        } else {
            args.snap = nullptr;
        }
    }
    return launch(kernel, grid, block, bytes, stream, args);
}

template <typename T, int MODE>
cudaError_t launch_gated_t(const GatedArgs& a, int n_seqs, int most_threads, cudaStream_t stream) {
    // 8 rows a thread: the G = dim / 8 warps of a column block work side by side and meet only where the recurrence needs
    // the whole column (the delta rule's S^T k, once a token)
    // (measured on a B200 at 16 heads of 128 x 256, 2,048 tokens: 16 rows a thread 2.8 / 1.8 ms (delta rule / matrix memory),
    // 8 rows 2.0 / 1.15 ms, 4 rows 2.9 / 1.13 ms: more warps hide the chain of multiply-adds, until the meeting of 32 warps costs more)
    return launch_gated_kd<T, kRows, MODE>(a, n_seqs, most_threads > 0 ? 256 : 0, stream);
}

}  // namespace

cudaError_t launch_gated_delta_scan(int dtype, const void* y, int stride, int q_col, int k_col, int v_col, int b_col, int a_col,
                                    const float* conv_q, const float* conv_k, const float* conv_v, int taps, const float* a_log,
                                    const float* dt_bias, float key_eps, float q_scale, float* state, int state_rows, const float* tail,
                                    const int* cu_q, const int* rows, int n_seqs, float* out, int heads, int kv_heads, int dim, int v_dim,
                                    int most_threads, int* status, cudaStream_t stream) {
    if (n_seqs == 0) return cudaSuccess;
    if (dim > 512 || taps < 1 || taps > 16 || kv_heads < 1 || heads % kv_heads) return cudaErrorInvalidValue;
    GatedArgs a = {};
    a.y = y; a.stride = stride; a.q_col = q_col; a.k_col = k_col; a.v_col = v_col; a.g1_col = b_col; a.g2_col = a_col;
    a.conv_q = conv_q; a.conv_k = conv_k; a.conv_v = conv_v; a.taps = taps; a.p1 = a_log; a.p2 = dt_bias;
    a.c1 = key_eps; a.c2 = q_scale; a.c3 = 0.f; a.state = state; a.state_rows = state_rows; a.tail = taps > 1 ? tail : nullptr;
    a.tail_channels = 2 * kv_heads * dim + heads * v_dim; a.cu_q = cu_q; a.rows = rows; a.out = out;
    a.heads = heads; a.kv_heads = kv_heads; a.dim = dim; a.v_dim = v_dim; a.status = status;
    return dtype == kBF16 ? launch_gated_t<__nv_bfloat16, 0>(a, n_seqs, most_threads, stream)
                          : launch_gated_t<float, 0>(a, n_seqs, most_threads, stream);
}

cudaError_t launch_memory_scan(int dtype, const void* y, int stride, int q_col, int k_col, int v_col, int i_col, int f_col,
                               const float* i_bias, const float* f_bias, float gate_cap, float q_scale, float den_eps, float* state,
                               int state_rows, const int* cu_q, const int* rows, int n_seqs, float* out, int heads, int dim, int v_dim,
                               int most_threads, int* status, cudaStream_t stream, float* snap) {
    if (n_seqs == 0) return cudaSuccess;
    if (dim > 512 || !(gate_cap > 0.f)) return cudaErrorInvalidValue;
    GatedArgs a = {};
    a.y = y; a.stride = stride; a.q_col = q_col; a.k_col = k_col; a.v_col = v_col; a.g1_col = i_col; a.g2_col = f_col;
    a.taps = 1; a.p1 = i_bias; a.p2 = f_bias; a.c1 = gate_cap; a.c2 = q_scale; a.c3 = den_eps;
    a.state = state; a.state_rows = state_rows; a.cu_q = cu_q; a.rows = rows; a.out = out;
    a.heads = heads; a.kv_heads = heads; a.dim = dim; a.v_dim = v_dim; a.status = status; a.snap = snap;
    return dtype == kBF16 ? launch_gated_t<__nv_bfloat16, 1>(a, n_seqs, most_threads, stream)
                          : launch_gated_t<float, 1>(a, n_seqs, most_threads, stream);
}

// ------------------------------------------------------------------------- the kept inputs of a short convolution

// One block a sequence, a thread a channel: slot i of the kept inputs takes input number (last - kept + 1 + i) of the
// request, which is a token of this step or, where the step brought fewer than `kept` tokens, an older slot.  A thread
// reads slot i + n after it has written the slots below i only, so the shift is safe in place.
template <typename T>
__global__ void conv_tail_kernel(const T* __restrict__ y, int stride, int c0, int w0, int c1, int w1, int c2, int w2, int c3, int w3,
                                 float* __restrict__ tail, int state_rows, int kept, int channels, const int* __restrict__ cu_q,
                                 const int* __restrict__ rows, int* status) {
    pdl_launch();
    pdl_wait();
    const int seq = blockIdx.x;
    const int t0 = cu_q[seq], t1 = cu_q[seq + 1];
    if (t1 <= t0) return;
    const int row = rows[seq];
    if (row < 0 || row >= state_rows) {
        if (threadIdx.x == 0 && blockIdx.y == 0) set_status(status, kStatusBadRow, row);
        return;
    }
    const int n = t1 - t0;
    for (int ch = blockIdx.y * blockDim.x + threadIdx.x; ch < channels; ch += gridDim.y * blockDim.x) {
        int col = ch < w0 ? c0 + ch : (ch < w0 + w1 ? c1 + ch - w0 : (ch < w0 + w1 + w2 ? c2 + ch - w0 - w1 : c3 + ch - w0 - w1 - w2));
        float* tr = tail + (size_t)row * kept * channels + ch;
        for (int i = 0; i < kept; ++i) {
            const int s = t1 - kept + i;
            tr[(size_t)i * channels] = s >= t0 ? to_float(y[(size_t)s * stride + col]) : tr[(size_t)(i + n) * channels];
        }
    }
}

cudaError_t launch_conv_tail_update(int dtype, const void* y, int stride, int c0, int w0, int c1, int w1, int c2, int w2, int c3, int w3,
                                    float* tail, int state_rows, int kept, int channels, const int* cu_q, const int* rows, int n_seqs,
                                    int* status, cudaStream_t stream) {
    if (n_seqs == 0 || channels == 0 || kept == 0) return cudaSuccess;
    const dim3 grid(n_seqs, max(1, min(64, (channels + 255) / 256)));
    if (dtype == kBF16)
        return launch(conv_tail_kernel<__nv_bfloat16>, grid, 256, 0, stream, (const __nv_bfloat16*)y, stride, c0, w0, c1, w1, c2, w2, c3, w3,
                      tail, state_rows, kept, channels, cu_q, rows, status);
    return launch(conv_tail_kernel<float>, grid, 256, 0, stream, (const float*)y, stride, c0, w0, c1, w1, c2, w2, c3, w3, tail, state_rows,
                  kept, channels, cu_q, rows, status);
}

// ------------------------------------------------------------------------- results normed before they are added

// One block a token: the mean squares of the parts' rows (a block sum each, in a fixed order), then
// out = sum_i s_i w_i p_i rsqrt(ms_i + eps), all in 32-bit.
__global__ void __launch_bounds__(256)
normed_sum_kernel(int n, const float* __restrict__ p0, const float* __restrict__ p1, const float* __restrict__ p2,
                  const float* __restrict__ p3, const float* __restrict__ w0, const float* __restrict__ w1,
                  const float* __restrict__ w2, const float* __restrict__ w3, float s0, float s1, float s2, float s3, float eps,
                  float* __restrict__ out, int width) {
    __shared__ float scratch[32];
    pdl_launch();
    pdl_wait();
    const size_t at = (size_t)blockIdx.x * width;
    const float* p[4] = {p0, p1, p2, p3};
    const float* w[4] = {w0, w1, w2, w3};
    const float s[4] = {s0, s1, s2, s3};
    float f[4] = {0.f, 0.f, 0.f, 0.f};
    for (int b = 0; b < n; ++b) {
        float ss = 0.f;
        for (int i = threadIdx.x; i < width; i += blockDim.x) { const float v = p[b][at + i]; ss = fmaf(v, v, ss); }
        f[b] = s[b] * rsqrtf(block_sum(ss, scratch) / (float)width + eps);
    }
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        float o = 0.f;
        for (int b = 0; b < n; ++b) o = fmaf(f[b] * w[b][i], p[b][at + i], o);
        out[at + i] = o;
    }
}

cudaError_t launch_normed_sum(int n, const float* p0, const float* p1, const float* p2, const float* p3, const float* w0, const float* w1,
                              const float* w2, const float* w3, float s0, float s1, float s2, float s3, float eps, float* out,
                              int n_tokens, int width, cudaStream_t stream) {
    if (n_tokens == 0) return cudaSuccess;
    if (n < 1 || n > 4) return cudaErrorInvalidValue;
    return launch(normed_sum_kernel, n_tokens, 256, 0, stream, n, p0, p1, p2, p3, w0, w1, w2, w3, s0, s1, s2, s3, eps, out, width);
}

__global__ void add_rows_kernel(float* __restrict__ x, const float* __restrict__ other, long long n) {
    pdl_launch();
    pdl_wait();
    for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < n; e += (long long)gridDim.x * blockDim.x) x[e] += other[e];
}

cudaError_t launch_add_rows(float* x, const float* other, long long n, cudaStream_t stream) {
    if (n == 0) return cudaSuccess;
    const int blocks = (int)min((n + 255) / 256, (long long)148 * 16);
    return launch(add_rows_kernel, blocks, 256, 0, stream, x, other, n);
}

}  // namespace vtb
