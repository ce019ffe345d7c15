// Mixers that carry a matrix of fixed size for each (request, head): gated linear attention and the generalized
// delta rule, and the norm-and-gate step that follows them.
//
// The recurrences, for one head with state S [dim, v_dim] in 32-bit:
//   gated linear attention   S <- diag(alpha_t) S + k_t v_t^T,                         o_t = S^T q_t
//   delta rule               S <- diag(w_t) S - (a_t * u_t)(u_t^T S_old) + k_t v_t^T,  o_t = S^T r_t
//   retention                S <- decay_h S + (k_t / sqrt(dim)) v_t^T,                  o_t = S^T q_t   (q, k rotated)
// Column j of S depends on column j alone, so a warp owns 32 columns of one (sequence, head) and walks the step's
// tokens of that sequence in order: a decoded token and a portion of a prompt are the same loop.  A thread keeps
// KD rows of its column in registers; the rows are spread over `G` threads a column (G warps), whose partial dot
// products meet in shared memory and are added in the order of g.  What enters the recurrence is formed in 32-bit while a batch of
// tokens is staged in shared memory: the decay from its low-rank gate (log-sigmoid and exp, or sigmoid and exp), the
// removal rate, the unit key.  The sums' order depends on dim alone, never on how the tokens were cut into steps.
#include "common.cuh"
#include "kernels.h"
#include "launch.cuh"

namespace vtb {

namespace {

constexpr int kScanCols = 32;     // columns of the state a warp owns
// Most threads of a CTA, by the rows a thread keeps in registers.  A CTA that holds all of a head's columns forms the
// gates once for all of them, which is what a step of many sequences with a token each wants; a long walk of few
// sequences wants the head's column blocks on several SMs instead (each then forms the gates again, and issues a
// quarter of the walk's instructions): the caller bounds the threads by the step's shape (`most_threads`).
constexpr int scan_threads(int kd) { return kd <= 32 ? 1024 : (kd <= 64 ? 512 : 256); }
constexpr int kScanTokens = 16;   // tokens staged in shared memory at once
// values of a token that a thread fetches through its fixed shares (the more threads a CTA has, the fewer each needs)
constexpr int scan_values(int kd) { return kd <= 32 ? 2 : (kd <= 64 ? 4 : 8); }

struct ScanArgs {
    const void* y;                // [tokens, stride]: the projections
    int stride;
    int q_col, k_col, v_col;      // q (or r), k, v
    int a_col;                    // delta rule: the removal rate's projection
    int low_col, rank;            // the low-rank gate's input
    const float* w2;              // [heads * dim, rank]
    const float* bias2;           // [heads * dim]: bias of the low-rank gate
    const float* a_bias;          // [heads * dim] (delta rule)
    float c1;                     // gated linear attention: 1 / tau;  delta rule: the decay's rate
    float c2;                     // gated linear attention: the scale of q;  delta rule: eps of the unit key
    float* state;                 // [state rows, heads, dim, v_dim]
    int state_rows;
    const int* cu_q;              // [sequences + 1]
    const int* rows;              // [sequences]
    float* out;                   // [tokens, heads * v_dim]
    int heads, dim, v_dim, groups;
    int col_blocks;               // warps of columns in a CTA
    int most_threads;             // > 0: the step is a long walk of few sequences (CTAs of 256 threads); 0: the kernel's own bound
    int* status;
    // retention (Fixed): bias2 holds one decay for each head, c2 scales k, and q and k are rotated while they are staged
    const float* freq;            // [half]: pairs (i, i + half) of a head's q and k turn by positions[t] * freq[i]
    int half;
    const int* positions;         // [tokens]
    // retention, a long walk cut into segments that run side by side: a "sequence" whose row is -(n + 1) starts from a
    // state of zeros and leaves its last state in ends[n] instead of a request's row
    float* ends;                  // [end rows, heads, dim, v_dim]
    int end_rows;
    int act;                      // 1: q, k and v pass through silu (in 32-bit) while they are staged; 0: as they are
};

__device__ __forceinline__ float log_sigmoid(float z) {
    // log(1 / (1 + exp(-z))) without overflow on either side
    return z < 0.f ? z - log1pf(expf(z)) : -log1pf(expf(-z));
}

__device__ __forceinline__ float sigmoid(float z) { return 1.f / (1.f + expf(-z)); }

// A CTA owns `col_blocks` * 32 columns of one (sequence, head): thread (c, g, cb) keeps rows [g KD, (g + 1) KD) of column
// (blockIdx.z col_blocks + cb) 32 + c in registers.  The step's tokens of the sequence are staged in batches of 16: all
// threads fetch the batch's projections (each thread the same columns of every token, four tokens' loads in flight at
// once), form decay, removal rate and unit key from them once for all columns, and then walk the batch's tokens out of
// shared memory.
// Walk: the variant for long walks of few sequences, compiled for CTAs of 256 threads (and the registers they may have).
// Fixed: retention.  No gate: the decay is one number a head, k (not q) carries the scale, and the staged q and k are
// rotated in 32-bit where they lie in shared memory.
template <typename T, int KD, bool Delta, bool Walk, bool Fixed>
__global__ void __launch_bounds__(Walk ? 256 : scan_threads(KD), (Walk && Fixed && KD <= 16) ? 3 : 1)
scan_kernel(const ScanArgs a) {
    extern __shared__ __align__(16) float smem[];
    pdl_launch();
    const int seq = blockIdx.x, h = blockIdx.y;
    const int c = threadIdx.x, g = threadIdx.y, cb = threadIdx.z;
    const int G = a.groups, CB = a.col_blocks;
    constexpr int TB = kScanTokens;
    constexpr int kScanValues = scan_values(KD);
    const int tid = (cb * G + g) * kScanCols + c, n_threads = kScanCols * G * CB;
    const int dim = a.dim, v_dim = a.v_dim, rank = a.rank;
    const int dim_p = G * KD, cols = CB * kScanCols;
    const int col0 = blockIdx.z * cols;
    const int j = col0 + cb * kScanCols + c;
    const bool col_ok = j < v_dim;
    constexpr int kVectors = Delta ? 3 : 2;                 // q (r), k and, for the delta rule, the removal rate
    const int per = kVectors * dim_p + rank + cols;         // values of a token that the CTA reads
    // shared memory: the low-rank gate's second matrix for this head; a batch of tokens; the meeting place of the groups
    float* w2s = smem;                                      // [dim, rank]
    float* low = w2s + ((dim * rank + 3) & ~3);             // [tokens, rank]
    float* qs = low + ((TB * rank + 3) & ~3);               // [tokens, dim_p] each:
    float* ks = qs + TB * dim_p;
    float* bs = ks + TB * dim_p;                            // delta rule: the removal rate, then that times the unit key
    float* ds = bs + (Delta ? TB * dim_p : 0);              // the decay
    float* us = ds + TB * dim_p;                            // delta rule: the unit key
    float* vs = us + (Delta ? TB * dim_p : 0);              // [tokens, cols]
    float* red = vs + TB * cols;                            // [2, CB, G, 32]: where the groups of a column meet inside a token
    float* op = red + 2 * CB * G * kScanCols;               // [tokens, G, cols]: the groups' shares of the outputs
    // the weights are written by no kernel of the step: they are read before the wait
    for (int e = tid; e < dim * rank; e += n_threads) w2s[e] = a.w2[(size_t)h * dim * rank + e];
    pdl_wait();
    const int t0 = a.cu_q[seq], t1 = a.cu_q[seq + 1];
    if (t1 <= t0) return;                                   // a sequence without tokens in this step (padding): its state stays
    const int row = a.rows[seq];
    const bool later = Fixed && row < 0 && a.ends != nullptr;      // a later segment of a walk that was cut
    if (later ? (-row - 1 >= a.end_rows) : (row < 0 || row >= a.state_rows)) {
        if (tid == 0) set_status(a.status, kStatusBadRow, row);
        return;
    }
    const T* y = reinterpret_cast<const T*>(a.y);
    // value r of a token: q, k, (removal rate), the gate's input, v
    auto fetch = [&](const T* yr, int r) -> float {
        if (r < kVectors * dim_p) {
            const int which = r < dim_p ? 0 : (r < 2 * dim_p ? 1 : 2), i = r - which * dim_p;
            if (i >= dim) return 0.f;
            const int col = which == 0 ? a.q_col : (which == 1 ? a.k_col : a.a_col);
            float v = to_float(yr[col + h * dim + i]);
            if (Fixed && a.act) v = v / (1.f + expf(-v));
            return (!Delta && which == (Fixed ? 1 : 0)) ? v * a.c2 : v;
        }
        r -= kVectors * dim_p;
        if (r < rank) {
            const float v = to_float(yr[a.low_col + r]);
            return Delta ? tanhf(v) : v;
        }
        r -= rank;
        if (col0 + r >= v_dim) return 0.f;
        const float v = to_float(yr[a.v_col + h * v_dim + col0 + r]);
        return (Fixed && a.act) ? v / (1.f + expf(-v)) : v;
    };
    auto place = [&](int tb, int r, float v) {
        if (r < kVectors * dim_p) {
            const int which = r < dim_p ? 0 : (r < 2 * dim_p ? 1 : 2);
            (which == 0 ? qs : (which == 1 ? ks : bs))[tb * dim_p + r - which * dim_p] = v;
            return;
        }
        r -= kVectors * dim_p;
        if (r < rank) { low[tb * rank + r] = v; return; }
        vs[tb * cols + r - rank] = v;
    };

    // Which of a token's values this thread fetches is the same for every token: value r = tid + k * threads comes from
    // column from_col[k] of the token's row (-1: padding, nothing to load), is multiplied by times[k] and lands at
    // smem[to_at[k] + token * to_step[k]] (-1: no such value).
    int from_col[kScanValues], to_at[kScanValues], to_step[kScanValues];
    float times[kScanValues];
    bool is_low[kScanValues];
#pragma unroll
    for (int k = 0; k < kScanValues; ++k) {
        int r = tid + k * n_threads;
        from_col[k] = -1; to_at[k] = -1; to_step[k] = 0; times[k] = 1.f; is_low[k] = false;
        if (r >= per) continue;
        if (r < kVectors * dim_p) {
            const int which = r < dim_p ? 0 : (r < 2 * dim_p ? 1 : 2), i = r - which * dim_p;
            to_at[k] = (int)((which == 0 ? qs : (which == 1 ? ks : bs)) - smem) + i;
            to_step[k] = dim_p;
            if (i < dim) from_col[k] = (which == 0 ? a.q_col : (which == 1 ? a.k_col : a.a_col)) + h * dim + i;
            if (!Delta && which == (Fixed ? 1 : 0)) times[k] = a.c2;
            continue;
        }
        r -= kVectors * dim_p;
        if (r < rank) {
            to_at[k] = (int)(low - smem) + r; to_step[k] = rank; from_col[k] = a.low_col + r; is_low[k] = true;
            continue;
        }
        r -= rank;
        to_at[k] = (int)(vs - smem) + r; to_step[k] = cols;
        if (col0 + r < v_dim) from_col[k] = a.v_col + h * v_dim + col0 + r;
    }

    float* sp = later ? a.ends + (((size_t)(-row - 1) * a.heads + h) * dim) * v_dim
                      : a.state + (((size_t)row * a.heads + h) * dim) * v_dim;
    float S[KD];
#pragma unroll
    for (int i = 0; i < KD; ++i) {
        const int r = g * KD + i;
        S[i] = (col_ok && r < dim && !later) ? sp[(size_t)r * v_dim + j] : 0.f;
    }
    int meet = 0;
    for (int tb0 = t0; tb0 < t1; tb0 += TB) {
        const int n = min(TB, t1 - tb0);
        __syncthreads();                                    // the batch before is done with
        // four tokens' values at a time: loads that wait for nothing but memory (the whole batch at once was measured and
        // was no faster: a prompt's portion 5 % slower, a decode step's scan 35 %)
        constexpr int kAtOnce = 4;
        for (int tb = 0; tb < n; tb += kAtOnce) {
            float val[kAtOnce][kScanValues];
#pragma unroll
            for (int u = 0; u < kAtOnce; ++u) {
                const T* yr = y + (size_t)(tb0 + min(tb + u, n - 1)) * a.stride;
#pragma unroll
                for (int k = 0; k < kScanValues; ++k) val[u][k] = from_col[k] >= 0 ? to_float(yr[from_col[k]]) : 0.f;
            }
#pragma unroll
            for (int u = 0; u < kAtOnce; ++u) {
                if (tb + u >= n) break;
#pragma unroll
                for (int k = 0; k < kScanValues; ++k) {
                    if (to_at[k] < 0) continue;
                    float v = val[u][k];
                    if (Fixed && a.act) v = v / (1.f + expf(-v));
                    v *= times[k];
                    if (Delta && is_low[k]) v = tanhf(v);
                    smem[to_at[k] + (tb + u) * to_step[k]] = v;
                }
            }
        }
        for (int tb = 0; tb < n; ++tb) {                    // sizes beyond what the threads' fixed shares cover
            const T* yr = y + (size_t)(tb0 + tb) * a.stride;
            for (int r = tid + kScanValues * n_threads; r < per; r += n_threads) place(tb, r, fetch(yr, r));
        }
        __syncthreads();
        if (Fixed) {
            const float decay = a.bias2[h];
            for (int e = tid; e < n * dim_p; e += n_threads) ds[e] = (e % dim_p) < dim ? decay : 0.f;
            // the rotation of q and k: a thread turns both members of a pair, so nothing else touches them meanwhile
            const int half = a.half;
            for (int e = tid; e < n * half; e += n_threads) {
                const int tb = e / half, i = e % half;
                const float angle = (float)a.positions[tb0 + tb] * a.freq[i];
                float sn, cs;
                sincosf(angle, &sn, &cs);
                float* qv = qs + tb * dim_p;
                float* kv = ks + tb * dim_p;
                const float qa = qv[i], qb = qv[i + half], ka = kv[i], kb = kv[i + half];
                qv[i] = qa * cs - qb * sn;
                qv[i + half] = qb * cs + qa * sn;
                kv[i] = ka * cs - kb * sn;
                kv[i + half] = kb * cs + ka * sn;
            }
        }
        for (int e = tid; !Fixed && e < n * dim_p; e += n_threads) {
            const int tb = e / dim_p, i = e % dim_p;
            float d = 0.f;
            if (i < dim) {
                const int ch = h * dim + i;
                float z = a.bias2[ch];
                const float* wr = w2s + i * rank;
                const float* lr = low + tb * rank;
                for (int r = 0; r < rank; ++r) z = fmaf(wr[r], lr[r], z);
                if (Delta) {
                    d = expf(-a.c1 * sigmoid(z));
                    bs[e] = sigmoid(bs[e] + a.a_bias[ch]);
                } else {
                    d = expf(a.c1 * log_sigmoid(z));
                }
            }
            ds[e] = d;
        }
        __syncthreads();
        if (Delta) {
            // the unit key u = k / sqrt(sum(k^2) + eps), and b = a * u: a warp for each staged token
            for (int tb = cb * G + g; tb < n; tb += G * CB) {
                float ss = 0.f;
                for (int i = c; i < dim_p; i += 32) ss = fmaf(ks[tb * dim_p + i], ks[tb * dim_p + i], ss);
                ss = warp_sum(ss);
                const float inv = 1.f / sqrtf(ss + a.c2);
                for (int i = c; i < dim_p; i += 32) {
                    const float u = ks[tb * dim_p + i] * inv;
                    us[tb * dim_p + i] = u;
                    bs[tb * dim_p + i] *= u;
                }
            }
            __syncthreads();
        }
        for (int tb = 0; tb < n; ++tb) {
            const float v = vs[tb * cols + cb * kScanCols + c];
            const float4* q4 = reinterpret_cast<const float4*>(qs + tb * dim_p + g * KD);
            const float4* k4 = reinterpret_cast<const float4*>(ks + tb * dim_p + g * KD);
            const float4* d4 = reinterpret_cast<const float4*>(ds + tb * dim_p + g * KD);
            float acc[4] = {0.f, 0.f, 0.f, 0.f};
            if (Delta) {
                const float4* u4 = reinterpret_cast<const float4*>(us + tb * dim_p + g * KD);
                const float4* b4 = reinterpret_cast<const float4*>(bs + tb * dim_p + g * KD);
                float part[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                for (int i = 0; i < KD / 4; ++i) {
                    const float4 u = u4[i];
                    part[0] = fmaf(u.x, S[4 * i + 0], part[0]);
                    part[1] = fmaf(u.y, S[4 * i + 1], part[1]);
                    part[2] = fmaf(u.z, S[4 * i + 2], part[2]);
                    part[3] = fmaf(u.w, S[4 * i + 3], part[3]);
                }
                float us_old = (part[0] + part[1]) + (part[2] + part[3]);
                if (G > 1) {
                    // u^T S of the old state is needed before the update: the G warps that share these columns meet
                    // (a barrier of their own; two buffers in turn, so one meeting a token is enough)
                    float* m = red + ((meet++ & 1) * CB + cb) * G * kScanCols;
                    m[g * kScanCols + c] = us_old;
                    asm volatile("bar.sync %0, %1;" ::"r"(cb + 1), "r"(G * kScanCols) : "memory");
                    us_old = 0.f;
                    for (int gg = 0; gg < G; ++gg) us_old += m[gg * kScanCols + c];
                }
#pragma unroll
                for (int i = 0; i < KD / 4; ++i) {
                    const float4 q = q4[i], k = k4[i], d = d4[i], b = b4[i];
                    S[4 * i + 0] = fmaf(d.x, S[4 * i + 0], fmaf(k.x, v, -b.x * us_old));
                    S[4 * i + 1] = fmaf(d.y, S[4 * i + 1], fmaf(k.y, v, -b.y * us_old));
                    S[4 * i + 2] = fmaf(d.z, S[4 * i + 2], fmaf(k.z, v, -b.z * us_old));
                    S[4 * i + 3] = fmaf(d.w, S[4 * i + 3], fmaf(k.w, v, -b.w * us_old));
                    acc[0] = fmaf(S[4 * i + 0], q.x, acc[0]);
                    acc[1] = fmaf(S[4 * i + 1], q.y, acc[1]);
                    acc[2] = fmaf(S[4 * i + 2], q.z, acc[2]);
                    acc[3] = fmaf(S[4 * i + 3], q.w, acc[3]);
                }
            } else {
#pragma unroll
                for (int i = 0; i < KD / 4; ++i) {
                    const float4 q = q4[i], k = k4[i], d = d4[i];
                    S[4 * i + 0] = fmaf(d.x, S[4 * i + 0], k.x * v);
                    S[4 * i + 1] = fmaf(d.y, S[4 * i + 1], k.y * v);
                    S[4 * i + 2] = fmaf(d.z, S[4 * i + 2], k.z * v);
                    S[4 * i + 3] = fmaf(d.w, S[4 * i + 3], k.w * v);
                    acc[0] = fmaf(S[4 * i + 0], q.x, acc[0]);
                    acc[1] = fmaf(S[4 * i + 1], q.y, acc[1]);
                    acc[2] = fmaf(S[4 * i + 2], q.z, acc[2]);
                    acc[3] = fmaf(S[4 * i + 3], q.w, acc[3]);
                }
            }
            // this group's share of the token's output: nothing of the recurrence waits for the sum over the groups,
            // which is formed once the batch is through
            op[(tb * G + g) * cols + cb * kScanCols + c] = (acc[0] + acc[1]) + (acc[2] + acc[3]);
        }
        __syncthreads();
        for (int e = tid; e < n * cols; e += n_threads) {
            const int tb = e / cols, cc = e % cols;
            if (col0 + cc >= v_dim) continue;
            float o = 0.f;
            for (int gg = 0; gg < G; ++gg) o += op[(tb * G + gg) * cols + cc];       // in the order of the groups
            a.out[(size_t)(tb0 + tb) * a.heads * v_dim + h * v_dim + col0 + cc] = o;
        }
    }
#pragma unroll
    for (int i = 0; i < KD; ++i) {
        const int r = g * KD + i;
        if (col_ok && r < dim) sp[(size_t)r * v_dim + j] = S[i];
    }
}

template <typename T, int KD, bool Delta, bool Walk, bool Fixed>
cudaError_t launch_scan_kd(ScanArgs a, int n_seqs, cudaStream_t stream) {
    static std::atomic<unsigned long long> done{0};
    const int G = a.groups, dim_p = G * KD;
    // as many warps of columns a CTA as the head has, within the CTA's threads
    const int col_warps = (a.v_dim + kScanCols - 1) / kScanCols;
    // (a group of warps that meets inside a token has a barrier of its own, of which a CTA has 15)
    const int threads = Walk ? min(256, scan_threads(KD)) : scan_threads(KD);
    const int most = max(1, min(threads / (kScanCols * G), G > 1 ? 15 : 32));
    const int ctas = (col_warps + most - 1) / most;                       // CTAs a head, with its warps of columns spread evenly
    a.col_blocks = (col_warps + ctas - 1) / ctas;
    const int cols = a.col_blocks * kScanCols;
    const size_t floats = ((a.dim * a.rank + 3) & ~3) + ((kScanTokens * a.rank + 3) & ~3)
                          + (size_t)(Delta ? 5 : 3) * kScanTokens * dim_p + kScanTokens * cols + 2 * a.col_blocks * G * kScanCols
                          + (size_t)kScanTokens * G * cols;
    const size_t bytes = floats * sizeof(float);
    constexpr int kMostBytes = 200 * 1024;
    if (bytes > kMostBytes) return cudaErrorInvalidValue;
    // the limit is set once for each device, so it is the most any launch may ask for, not what this one asks for
    cudaError_t e = allow_dynamic_smem(scan_kernel<T, KD, Delta, Walk, Fixed>, kMostBytes, done);
    if (e != cudaSuccess) return e;
    dim3 grid(n_seqs, a.heads, (col_warps + a.col_blocks - 1) / a.col_blocks), block(kScanCols, G, a.col_blocks);
    return launch(scan_kernel<T, KD, Delta, Walk, Fixed>, grid, block, bytes, stream, a);
}

template <typename T, bool Delta, bool Fixed = false>
cudaError_t launch_scan_t(ScanArgs a, int n_seqs, cudaStream_t stream) {
    // Rows a thread: 16 where that makes at most 8 groups of warps a column, else 32, 64, 128.  Few rows a thread make
    // the walk along the tokens short (a token costs a thread rows / 4 steps of loads and multiply-adds, whatever the
    // number of groups), which is what bounds a sequence's portion of a prompt; the groups' shares meet in shared memory.
    const int kd = a.dim <= 128 ? 16 : (a.dim <= 256 ? 32 : (a.dim <= 512 ? 64 : 128));
    a.groups = (a.dim + kd - 1) / kd;
    if (a.groups > 8) return cudaErrorInvalidValue;
    const bool walk = a.most_threads > 0;
    if (kd == 16) return walk ? launch_scan_kd<T, 16, Delta, true, Fixed>(a, n_seqs, stream) : launch_scan_kd<T, 16, Delta, false, Fixed>(a, n_seqs, stream);
    if (kd == 32) return walk ? launch_scan_kd<T, 32, Delta, true, Fixed>(a, n_seqs, stream) : launch_scan_kd<T, 32, Delta, false, Fixed>(a, n_seqs, stream);
    if (kd == 64) return walk ? launch_scan_kd<T, 64, Delta, true, Fixed>(a, n_seqs, stream) : launch_scan_kd<T, 64, Delta, false, Fixed>(a, n_seqs, stream);
    return launch_scan_kd<T, 128, Delta, false, Fixed>(a, n_seqs, stream);
}

}  // namespace

cudaError_t launch_gla_scan(int dtype, const void* y, int stride, int q_col, int k_col, int v_col, int low_col, int rank,
                            const float* a2, const float* a2_bias, float inv_tau, float q_scale, float* state,
                            int state_rows, const int* cu_q, const int* rows, int n_seqs, float* out, int heads, int dim,
                            int v_dim, int most_threads, int* status, cudaStream_t stream) {
    if (n_seqs == 0) return cudaSuccess;
    ScanArgs a = {y, stride, q_col, k_col, v_col, 0, low_col, rank, a2, a2_bias, nullptr, inv_tau, q_scale, state,
                  state_rows, cu_q, rows, out, heads, dim, v_dim, 1, 1, most_threads, status};
    return dtype == kBF16 ? launch_scan_t<__nv_bfloat16, false>(a, n_seqs, stream) : launch_scan_t<float, false>(a, n_seqs, stream);
}

cudaError_t launch_delta_scan(int dtype, const void* y, int stride, int r_col, int k_col, int v_col, int a_col, int low_col,
                              int rank, const float* w2, const float* w0, const float* a_bias, float decay_rate,
                              float key_eps, float* state, int state_rows, const int* cu_q, const int* rows, int n_seqs,
                              float* out, int heads, int dim, int most_threads, int* status, cudaStream_t stream) {
    if (n_seqs == 0) return cudaSuccess;
    ScanArgs a = {y, stride, r_col, k_col, v_col, a_col, low_col, rank, w2, w0, a_bias, decay_rate, key_eps, state,
                  state_rows, cu_q, rows, out, heads, dim, dim, 1, 1, most_threads, status};
    return dtype == kBF16 ? launch_scan_t<__nv_bfloat16, true>(a, n_seqs, stream) : launch_scan_t<float, true>(a, n_seqs, stream);
}

cudaError_t launch_retention_scan(int dtype, const void* y, int stride, int q_col, int k_col, int v_col, const float* decay,
                                  float k_scale, const float* freq, int half, const int* positions, float* state, int state_rows,
                                  const int* cu_q, const int* rows, int n_seqs, float* out, int heads, int dim, int v_dim,
                                  int most_threads, int* status, float* ends, int end_rows, cudaStream_t stream, int act) {
    if (n_seqs == 0) return cudaSuccess;
    if (2 * half > dim) return cudaErrorInvalidValue;
    // no low-rank gate (rank 0); the gate's bias slot carries the heads' decays, c2 the scale of k
    ScanArgs a = {y, stride, q_col, k_col, v_col, 0, 0, 0, nullptr, decay, nullptr, 0.f, k_scale, state, state_rows, cu_q, rows,
                  out, heads, dim, v_dim, 1, 1, most_threads, status, freq, half, positions, ends, end_rows, act};
    return dtype == kBF16 ? launch_scan_t<__nv_bfloat16, false, true>(a, n_seqs, stream)
                          : launch_scan_t<float, false, true>(a, n_seqs, stream);
}

// ------------------------------------------------------------------------- retention: a long walk cut into segments
//
// With one fixed decay a head the recurrence is linear in the state it starts from: a segment that starts from zeros
// gives each of its tokens the share of the segment's own keys, and what the state before the segment adds to token t
// is decay^(t - t0 + 1) S_before^T q_t.  So the segments of a long portion run side by side (the scan kernel, the
// first segment from the request's state, the later ones from zeros into `ends`); one kernel then carries the state
// from segment to segment (S_before of the next = decay^length S_before + end), leaving every later segment's
// S_before in `starts` and the last state in the request's row; and one adds the missing share to the later segments'
// outputs.  Everything in 32-bit; only the order of the sums differs from the walk in one piece.

// One thread an element of a (sequence, head)'s state; the sequence's later segments in order.
__global__ void __launch_bounds__(256)
retention_carry_kernel(float* __restrict__ state, int state_rows, const float* __restrict__ ends, float* __restrict__ starts,
                       const int* __restrict__ seq_row, const int* __restrict__ seq_first, const int* __restrict__ seq_count,
                       const int* __restrict__ seg_len, const float* __restrict__ decay, int heads, int per_head, int* status) {
    pdl_launch();
    pdl_wait();
    const int s = blockIdx.x, h = blockIdx.y;
    const int e = blockIdx.z * blockDim.x + threadIdx.x;
    if (e >= per_head) return;
    const int row = seq_row[s];
    if (row < 0 || row >= state_rows) {
        if (e == 0) set_status(status, kStatusBadRow, row);
        return;
    }
    const int first = seq_first[s], count = seq_count[s];
    const float g = decay[h];
    float* sp = state + ((size_t)row * heads + h) * per_head + e;
    float S = *sp;                                              // the state after the first segment
    for (int j = 0; j < count; ++j) {
        const size_t at = ((size_t)(first + j) * heads + h) * per_head + e;
        starts[at] = S;
        S = fmaf(powf(g, (float)seg_len[first + j]), S, ends[at]);
    }
    *sp = S;
}

// A tile of up to 32 tokens of a later segment, 128 columns of a head: out[t, j] += decay^(t - t0 + 1) sum_i q_t[i] S[i, j],
// q rotated as the scan rotates it.  The state's rows come 32 at a time into registers, the tokens' q into shared memory.
template <typename T>
__global__ void __launch_bounds__(128)
retention_fix_kernel(const T* __restrict__ y, int stride, int q_col, const int* __restrict__ positions, const float* __restrict__ freq,
                     int half, const float* __restrict__ starts, const int4* __restrict__ tiles, const float* __restrict__ decay,
                     float* __restrict__ out, int heads, int dim, int v_dim, int act) {
    constexpr int TT = 32, RR = 32;
    __shared__ __align__(16) float qs[TT][RR];
    pdl_launch();
    pdl_wait();
    const int4 tile = tiles[blockIdx.x];            // (later segment, first token of the tile, tokens, first token of the segment)
    const int seg = tile.x, t_begin = tile.y, n = tile.z, t0 = tile.w;
    const int h = blockIdx.y, j = blockIdx.z * blockDim.x + threadIdx.x;
    const bool col_ok = j < v_dim;
    const float* S = starts + ((size_t)seg * heads + h) * dim * v_dim;
    float acc[TT];
#pragma unroll
    for (int tk = 0; tk < TT; ++tk) acc[tk] = 0.f;
    for (int r0 = 0; r0 < dim; r0 += RR) {
        __syncthreads();
        for (int e = threadIdx.x; e < TT * RR; e += blockDim.x) {
            const int tk = e / RR, i = r0 + e % RR;
            float v = 0.f;
            if (tk < n && i < dim) {
                const T* qp = y + (size_t)(t_begin + tk) * stride + q_col + h * dim;
                auto value = [&](int at) {
                    const float z = to_float(qp[at]);
                    return act ? z / (1.f + expf(-z)) : z;       // as the scan stages it
                };
                v = value(i);
                if (i < 2 * half) {
                    const int f = i < half ? i : i - half;
                    float sn, cs;
                    sincosf((float)positions[t_begin + tk] * freq[f], &sn, &cs);
                    v = i < half ? v * cs - value(i + half) * sn : v * cs + value(i - half) * sn;
                }
            }
            qs[tk][e % RR] = v;
        }
        float Sr[RR];
#pragma unroll
        for (int i = 0; i < RR; ++i) Sr[i] = (col_ok && r0 + i < dim) ? S[(size_t)(r0 + i) * v_dim + j] : 0.f;
        __syncthreads();
#pragma unroll
        for (int tk = 0; tk < TT; ++tk) {
            const float4* q4 = reinterpret_cast<const float4*>(qs[tk]);
            float part[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int i = 0; i < RR / 4; ++i) {
                const float4 q = q4[i];
                part[0] = fmaf(q.x, Sr[4 * i + 0], part[0]);
                part[1] = fmaf(q.y, Sr[4 * i + 1], part[1]);
                part[2] = fmaf(q.z, Sr[4 * i + 2], part[2]);
                part[3] = fmaf(q.w, Sr[4 * i + 3], part[3]);
            }
            acc[tk] += (part[0] + part[1]) + (part[2] + part[3]);
        }
    }
    if (!col_ok) return;
    const float g = decay[h];
#pragma unroll
    for (int tk = 0; tk < TT; ++tk) {
        if (tk >= n) break;
        const int t = t_begin + tk;
        float* o = out + (size_t)t * heads * v_dim + h * v_dim + j;
        *o = fmaf(powf(g, (float)(t - t0 + 1)), acc[tk], *o);
    }
}

cudaError_t launch_retention_carry(float* state, int state_rows, const float* ends, float* starts, const int* seq_row,
                                   const int* seq_first, const int* seq_count, const int* seg_len, int n_split, const float* decay,
                                   int heads, int dim, int v_dim, int* status, cudaStream_t stream) {
    if (n_split == 0) return cudaSuccess;
    const int per_head = dim * v_dim;
    return launch(retention_carry_kernel, dim3(n_split, heads, (per_head + 255) / 256), 256, 0, stream, state, state_rows, ends, starts,
                  seq_row, seq_first, seq_count, seg_len, decay, heads, per_head, status);
}

cudaError_t launch_retention_fix(int dtype, const void* y, int stride, int q_col, const int* positions, const float* freq, int half,
                                 const float* starts, const int* tiles, int n_tiles, const float* decay, float* out, int heads, int dim,
                                 int v_dim, cudaStream_t stream, int act) {
    if (n_tiles == 0) return cudaSuccess;
    const dim3 grid(n_tiles, heads, (v_dim + 127) / 128);
    if (dtype == kBF16)
        return launch(retention_fix_kernel<__nv_bfloat16>, grid, 128, 0, stream, (const __nv_bfloat16*)y, stride, q_col, positions, freq,
                      half, starts, reinterpret_cast<const int4*>(tiles), decay, out, heads, dim, v_dim, act);
    return launch(retention_fix_kernel<float>, grid, 128, 0, stream, (const float*)y, stride, q_col, positions, freq, half, starts,
                  reinterpret_cast<const int4*>(tiles), decay, out, heads, dim, v_dim, act);
}

// ------------------------------------------------------------------------- norm of each head's output, gate

// One warp for a (token, head): out = out_scale * o / sqrt(mean(o^2) + eps) * w * act(gate), all in 32-bit.
template <typename T>
__global__ void __launch_bounds__(128)
head_norm_gate_kernel(const float* __restrict__ o, const T* __restrict__ y, int y_stride, int gate_col,
                      const float* __restrict__ weight, int weight_per_channel, float eps, int act, T* __restrict__ out,
                      int out_stride, int out_col, float out_scale, const int* __restrict__ token_seq, int n_tokens, int heads,
                      int v_dim) {
    pdl_launch();
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const long long pair = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (pair >= (long long)n_tokens * heads) return;
    const int t = (int)(pair / heads), h = (int)(pair % heads);
    T* dst = out + (size_t)t * out_stride + out_col + h * v_dim;
    if (token_seq != nullptr && token_seq[t] < 0) {     // padding: nothing ran for this token
        for (int i = lane; i < v_dim; i += 32) dst[i] = from_float<T>(0.f);
        return;
    }
    const float* src = o + ((size_t)t * heads + h) * v_dim;
    float ss = 0.f;
    for (int i = lane; i < v_dim; i += 32) ss = fmaf(src[i], src[i], ss);
    ss = warp_sum(ss);
    const float r = rsqrtf(ss / (float)v_dim + eps) * out_scale;
    const T* gate = y + (size_t)t * y_stride + gate_col + h * v_dim;
    const float* w = weight + (weight_per_channel ? h * v_dim : 0);
    for (int i = lane; i < v_dim; i += 32) {
        const float z = to_float(gate[i]);
        const float s = 1.f / (1.f + expf(-z));
        dst[i] = from_float<T>(src[i] * r * w[i] * (act == 0 ? z * s : s));
    }
}

// The same for heads of many values (heads normed together are one head as wide as all of them): a CTA a (token, head),
// its warps' sums of squares added in the order of the warps.
template <typename T>
__global__ void __launch_bounds__(256)
head_norm_gate_wide_kernel(const float* __restrict__ o, const T* __restrict__ y, int y_stride, int gate_col,
                           const float* __restrict__ weight, int weight_per_channel, float eps, int act, T* __restrict__ out,
                           int out_stride, int out_col, float out_scale, const int* __restrict__ token_seq, int heads, int v_dim) {
    __shared__ float sums[8];
    pdl_launch();
    pdl_wait();
    const int t = blockIdx.x / heads, h = blockIdx.x % heads;
    T* dst = out + (size_t)t * out_stride + out_col + h * v_dim;
    if (token_seq != nullptr && token_seq[t] < 0) {     // padding: nothing ran for this token
        for (int i = threadIdx.x; i < v_dim; i += 256) dst[i] = from_float<T>(0.f);
        return;
    }
    const float* src = o + ((size_t)t * heads + h) * v_dim;
    float ss = 0.f;
    for (int i = threadIdx.x; i < v_dim; i += 256) ss = fmaf(src[i], src[i], ss);
    ss = warp_sum(ss);
    if ((threadIdx.x & 31) == 0) sums[threadIdx.x >> 5] = ss;
    __syncthreads();
    float total = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) total += sums[k];
    const float r = rsqrtf(total / (float)v_dim + eps) * out_scale;
    const T* gate = y + (size_t)t * y_stride + gate_col + h * v_dim;
    const float* w = weight + (weight_per_channel ? h * v_dim : 0);
    for (int i = threadIdx.x; i < v_dim; i += 256) {
        const float z = to_float(gate[i]);
        const float sg = 1.f / (1.f + expf(-z));
        dst[i] = from_float<T>(src[i] * r * w[i] * (act == 0 ? z * sg : sg));
    }
}

cudaError_t launch_head_norm_gate(int dtype, const float* o, const void* y, int y_stride, int gate_col, const float* weight,
                                  int weight_per_channel, float eps, int act, void* out, int out_stride, int out_col,
                                  float out_scale, const int* token_seq, int n_tokens, int heads, int v_dim, cudaStream_t stream) {
    const long long pairs = (long long)n_tokens * heads;
    if (pairs == 0) return cudaSuccess;
    if (v_dim >= 1024) {
        if (dtype == kBF16)
            return launch(head_norm_gate_wide_kernel<__nv_bfloat16>, (int)pairs, 256, 0, stream, o, (const __nv_bfloat16*)y, y_stride,
                          gate_col, weight, weight_per_channel, eps, act, (__nv_bfloat16*)out, out_stride, out_col, out_scale, token_seq,
                          heads, v_dim);
        return launch(head_norm_gate_wide_kernel<float>, (int)pairs, 256, 0, stream, o, (const float*)y, y_stride, gate_col, weight,
                      weight_per_channel, eps, act, (float*)out, out_stride, out_col, out_scale, token_seq, heads, v_dim);
    }
    const int blocks = (int)((pairs + 3) / 4);
    if (dtype == kBF16)
        return launch(head_norm_gate_kernel<__nv_bfloat16>, blocks, 128, 0, stream, o, (const __nv_bfloat16*)y, y_stride, gate_col,
                      weight, weight_per_channel, eps, act, (__nv_bfloat16*)out, out_stride, out_col, out_scale, token_seq,
                      n_tokens, heads, v_dim);
    return launch(head_norm_gate_kernel<float>, blocks, 128, 0, stream, o, (const float*)y, y_stride, gate_col, weight,
                  weight_per_channel, eps, act, (float*)out, out_stride, out_col, out_scale, token_seq, n_tokens, heads, v_dim);
}

}  // namespace vtb
