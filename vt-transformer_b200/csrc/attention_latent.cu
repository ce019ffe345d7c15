// Softmax attention over paged rows that all heads share, on the tensor cores (bfloat16 in, 32-bit softmax and sums).
//
// A token keeps one row of D numbers (a latent of DV numbers and a key part of D - DV numbers behind it).  Every head's
// key is the whole row and every head's value the row's first DV numbers, so the heads of a token differ in their
// queries only (the caller has taken them into the row's space): out[t, h] = sum_j p_j row_j[:DV],
// p = softmax_j(scale q_{t,h} . row_j) over the keys j <= position of t.  With sinks the softmax's denominator also
// holds exp(sink_h): a term without a key and without a value, not scaled.
//
// A tile is 64 rows of (token, head): a block of keys is brought into shared memory once for all of them (two-stage
// cp.async pipeline), and serves as K in S = Q K^T and, its first DV columns read transposed, as V in O += P V (mma.sync
// m16n8k16, P rounded to bfloat16).  The queries of the tile stay in shared memory (a row of D numbers does not fit the
// registers).  A slab of 16 rows has two warps (or four); each forms the slab's scores over its share of the D inner
// numbers, they add each other's shares through shared memory in a fixed order (so all hold the same scores, maxima and
// sums), and each owns its share of the columns of O.  The sink is where the running maximum and sum start: m = sink, l = 1.
// Prompt portions and single tokens run the same kernel (a single token's tile holds its heads).
#include "attention_mma.cuh"
#include "common.cuh"
#include "kernels.h"
#include "launch.cuh"

namespace vtb {

struct LatentParams {
    const __nv_bfloat16* q;          // [tokens, q_stride]: head h's query at q_col + h * D
    int q_stride, q_col;
    __nv_bfloat16* out;              // [tokens, out_stride]: head h's result at out_col + h * DV
    int out_stride, out_col;
    const __nv_bfloat16* pages;      // [pages, 1, page_size, D]
    const int* cu_q;
    const int* q_start;
    const int* block_table;
    int table_stride;
    const int2* tiles;               // (sequence, first token of the tile among the sequence's new tokens); null: a step of
                                     // single tokens, tile = sequence = token
    int n_pages, heads, page_size;
    int D, DV;                       // multiples of 16
    float scale_log2;                // scale * log2(e)
    const float* sinks;              // [heads] or null
    int tokens_per_tile, heads_per_tile;
    // a step of single tokens may cut every sequence's keys into n_splits runs of blocks, a CTA each (blockIdx.z): the runs
    // leave their unnormalised sums, maxima and sums in part [n_splits, tokens, heads, DV + 2] and a second kernel merges them
    int n_splits, n_tokens;
    float* part;
};

namespace {

constexpr int LAT_ROWS = 64;

// DVT: the columns of O that the kernel has registers for (DV <= DVT); KBL: keys in a block; MINB: CTAs an SM that the
// registers are to leave room for (values of up to 256 numbers fit two CTAs of 128 registers a thread: four warps a
// scheduler instead of two hide more of the fragment loads' and the products' latency).
template <int DVT, int KBL, int MINB, int WPS>
__global__ void __launch_bounds__(128 * WPS, MINB)
attention_latent_kernel(const LatentParams p) {
    constexpr int WARPS = 4 * WPS;            // four slabs of 16 rows, WPS warps a slab
    constexpr int THREADS = 32 * WARPS;
    constexpr int NJ = KBL / 8;               // tiles of 8 keys of a block
    constexpr int NK = KBL / 16;              // steps of 16 keys in the product with the values
    constexpr int HALF = DVT / WPS;           // columns of O that a warp owns
    constexpr int ND = HALF / 16;             // steps of 16 of them
    const int D = p.D, DV = p.DV, LD = D + 8; // padded rows: conflict-free fragment loads, 16-byte aligned
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __nv_bfloat16* qs = reinterpret_cast<__nv_bfloat16*>(smem_raw);   // [64][LD]
    __nv_bfloat16* ks = qs + (size_t)LAT_ROWS * LD;                   // [2 stages][KBL][LD]
    float4* xch = reinterpret_cast<float4*>(ks + (size_t)2 * KBL * LD); // [8 warps][NJ][32 lanes]: a pair's halves of the scores

    pdl_launch();
    pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, gq = lane >> 2, tq = lane & 3;
    const int rg = warp / WPS, side = warp % WPS, col0 = side * HALF;
    // the pair's warps form the slab's scores over one half of the D inner numbers each and add the other's half
    const int ks_per = (D / 16 + WPS - 1) / WPS;
    const int ks_lo = min(D / 16, side * ks_per), ks_hi = min(D / 16, ks_lo + ks_per);
    const int head0 = blockIdx.y * p.heads_per_tile;
    const int nheads = min(p.heads_per_tile, p.heads - head0);
    int seq = blockIdx.x, tok0 = 0;
    if (p.tiles) {
        const int2 tile = p.tiles[blockIdx.x];
        seq = tile.x;
        tok0 = tile.y;
    }
    const int q_begin = p.cu_q[seq];
    const int q_len = p.cu_q[seq + 1] - q_begin;
    const int ntok = min(p.tokens_per_tile, q_len - tok0);
    if (ntok <= 0) {
        // a step of single tokens padded to a captured graph's size: sequence i without a token is padding token i,
        // whose row of the result is cleared so that what follows reads numbers
        if (!p.tiles) {
            __nv_bfloat16* op = p.out + (size_t)blockIdx.x * p.out_stride + p.out_col + (size_t)head0 * DV;
            for (int e = threadIdx.x; e < nheads * DV; e += THREADS) op[e] = __float2bfloat16_rn(0.f);
        }
        return;
    }
    const int rows_valid = ntok * p.heads_per_tile;    // rows of heads beyond the last head are dead inside
    const int row_base = rg * 16;
    const bool slab_live = row_base < rows_valid;
    const int pos_lo = p.q_start[seq] + tok0, pos_hi = pos_lo + ntok - 1;
    const int key_hi = pos_hi + 1;
    const int nblk = (key_hi + KBL - 1) / KBL;
    int blk_lo = 0, blk_hi = nblk;
    if (p.n_splits > 1) {
        const int per = (nblk + p.n_splits - 1) / p.n_splits;
        blk_lo = min(nblk, (int)blockIdx.z * per);
        blk_hi = min(nblk, blk_lo + per);
    }

    // the two rows of this thread
    int pos[2], tok[2], head[2];
    bool valid[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int row = row_base + gq + 8 * i;
        const int tk = row / p.heads_per_tile, hh = row % p.heads_per_tile;
        valid[i] = tk < ntok && hh < nheads;
        tok[i] = q_begin + tok0 + (valid[i] ? tk : 0);
        pos[i] = pos_lo + (valid[i] ? tk : 0);
        head[i] = head0 + (valid[i] ? hh : 0);
    }

    const int KC = D / 8;                              // 16-byte pieces in a row
    // the tile's queries: a warp a row at a time
    for (int r = warp; r < LAT_ROWS; r += WARPS) {
        const int tk = r / p.heads_per_tile, hh = r % p.heads_per_tile;
        const bool ok = tk < ntok && hh < nheads;
        const __nv_bfloat16* src = p.q + (size_t)(q_begin + tok0 + (ok ? tk : 0)) * p.q_stride + p.q_col + (size_t)(head0 + (ok ? hh : 0)) * D;
        for (int c = lane; c < KC; c += 32) cp_async16(qs + (size_t)r * LD + c * 8, src + c * 8, ok);
    }
    const int* table = p.block_table + (size_t)seq * p.table_stride;
    auto load_block = [&](int blk, int stage) {
        const int kb = blk * KBL;
        for (int r = warp; r < KBL; r += WARPS) {
            const int key = kb + r;
            bool ok = key < key_hi;
            size_t base = 0;
            if (ok) {
                const int page = table[key / p.page_size];
                ok = page >= 0 && page < p.n_pages;
                if (ok) base = ((size_t)page * p.page_size + key % p.page_size) * D;
            }
            __nv_bfloat16* dst = ks + ((size_t)stage * KBL + r) * LD;
            for (int c = lane; c < KC; c += 32) cp_async16(dst + c * 8, p.pages + base + c * 8, ok);
        }
    };

    float o[2 * ND][4];
#pragma unroll
    for (int i = 0; i < 2 * ND; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    // the sink is the first term of the softmax: the maximum starts at it and the sum at one (held by one of the four
    // lanes that share a row: the lanes' sums are added at the end)
    float mrow[2] = {-INFINITY, -INFINITY}, lrow[2] = {0.f, 0.f};
    if (p.sinks && blockIdx.z == 0) {
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            if (valid[i]) {
                mrow[i] = p.sinks[head[i]] * 1.4426950408889634f;
                lrow[i] = tq == 0 ? 1.f : 0.f;
            }
        }
    }

    if (blk_lo < blk_hi) load_block(blk_lo, 0);
    cp_async_commit();
    for (int blk = blk_lo; blk < blk_hi; ++blk) {
        const int stage = (blk - blk_lo) & 1;
        if (blk + 1 < blk_hi) load_block(blk + 1, stage ^ 1);
        cp_async_commit();
        cp_async_wait<1>();
        __syncthreads();
        if (!slab_live) {                                // a slab without rows (a short tile): copies and barriers only
            __syncthreads();
            continue;
        }
        const __nv_bfloat16* kst = ks + (size_t)stage * KBL * LD;
        const int kb = blk * KBL;

        // S = Q K^T
        float s[NJ][4];
#pragma unroll
        for (int j = 0; j < NJ; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
        {
            const __nv_bfloat16* qrow = qs + (size_t)(row_base + (lane & 7) + ((lane >> 3) & 1) * 8) * LD + (lane >> 4) * 8;
            const int mat = lane >> 3, r = lane & 7;
            const __nv_bfloat16* krow = kst + (size_t)((mat >> 1) * 8 + r) * LD + (mat & 1) * 8;
            for (int ks_ = ks_lo; ks_ < ks_hi; ++ks_) {
                uint32_t qf[4];
                ldmatrix_x4(qf, qrow + ks_ * 16);
#pragma unroll
                for (int j = 0; j < NJ; j += 2) {
                    uint32_t kf[4];
                    ldmatrix_x4(kf, krow + (size_t)j * 8 * LD + ks_ * 16);
                    mma_bf16(s[j], qf, kf[0], kf[1]);
                    mma_bf16(s[j + 1], qf, kf[2], kf[3]);
                }
            }
        }
        {
            float4* mine = xch + (size_t)warp * NJ * 32 + lane;
#pragma unroll
            for (int j = 0; j < NJ; ++j) mine[j * 32] = make_float4(s[j][0], s[j][1], s[j][2], s[j][3]);
            asm volatile("bar.sync %0, %1;\n" ::"r"(1 + rg), "n"(32 * WPS) : "memory");   // the warps of the slab
            if (WPS == 2) {
                const float4* theirs = xch + (size_t)(warp ^ 1) * NJ * 32 + lane;
#pragma unroll
                for (int j = 0; j < NJ; ++j) {                                    // a + b = b + a: both warps hold the same sums
                    const float4 t = theirs[j * 32];
                    s[j][0] += t.x; s[j][1] += t.y; s[j][2] += t.z; s[j][3] += t.w;
                }
            } else {
                // all parts in the order of the warps, the own one from shared memory too: every warp holds the same sums
#pragma unroll
                for (int j = 0; j < NJ; ++j) {
                    float4 a = xch[((size_t)(rg * WPS) * NJ + j) * 32 + lane];
#pragma unroll
                    for (int w = 1; w < WPS; ++w) {
                        const float4 t = xch[((size_t)(rg * WPS + w) * NJ + j) * 32 + lane];
                        a.x += t.x; a.y += t.y; a.z += t.z; a.w += t.w;
                    }
                    s[j][0] = a.x; s[j][1] = a.y; s[j][2] = a.z; s[j][3] = a.w;
                }
            }
        }
        // mask, running maximum and sum (log2 domain)
        float mnew[2] = {mrow[0], mrow[1]};
        const bool open = kb + KBL - 1 <= pos_lo && rows_valid >= row_base + 16 && nheads == p.heads_per_tile;
        if (open) {                                      // every row of the slab sees all of the block's keys
#pragma unroll
            for (int j = 0; j < NJ; ++j) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    s[j][e] *= p.scale_log2;
                    mnew[e >> 1] = fmaxf(mnew[e >> 1], s[j][e]);
                }
            }
        } else {
#pragma unroll
            for (int j = 0; j < NJ; ++j) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int i = e >> 1;
                    const int key = kb + j * 8 + 2 * tq + (e & 1);
                    s[j][e] = (valid[i] && key <= pos[i]) ? s[j][e] * p.scale_log2 : -INFINITY;
                    mnew[i] = fmaxf(mnew[i], s[j][e]);
                }
            }
        }
        float corr[2];
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            mnew[i] = fmaxf(mnew[i], __shfl_xor_sync(0xffffffffu, mnew[i], 1));
            mnew[i] = fmaxf(mnew[i], __shfl_xor_sync(0xffffffffu, mnew[i], 2));
            corr[i] = (mnew[i] == -INFINITY) ? 1.f : fast_exp2(mrow[i] - mnew[i]);
            mrow[i] = mnew[i];
            lrow[i] *= corr[i];
        }
        const float base[2] = {mnew[0] == -INFINITY ? 0.f : mnew[0], mnew[1] == -INFINITY ? 0.f : mnew[1]};
#pragma unroll
        for (int j = 0; j < NJ; ++j) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float pv = fast_exp2(s[j][e] - base[e >> 1]);   // 2^(-inf) = 0 for masked keys
                s[j][e] = pv;
                lrow[e >> 1] += pv;
            }
        }
        if (__any_sync(0xffffffffu, corr[0] != 1.f || corr[1] != 1.f)) {   // no maximum moved: nothing to rescale
#pragma unroll
            for (int i = 0; i < 2 * ND; ++i) {
                o[i][0] *= corr[0]; o[i][1] *= corr[0];
                o[i][2] *= corr[1]; o[i][3] *= corr[1];
            }
        }
        // O += P V: the values are the first DV columns of the keys' rows
#pragma unroll
        for (int kk = 0; kk < NK; ++kk) {
            uint32_t pf[4];
            pf[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
            pf[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
            pf[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
            pf[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
            const int mat = lane >> 3, r = lane & 7;
            const __nv_bfloat16* vrow = kst + (size_t)(kk * 16 + (mat & 1) * 8 + r) * LD + col0 + (mat >> 1) * 8;
#pragma unroll
            for (int dn = 0; dn < ND; ++dn) {
                if (col0 + dn * 16 < DV) {               // the same for all of the warp
                    uint32_t vf[4];
                    ldmatrix_x4_trans(vf, vrow + dn * 16);
                    mma_bf16(o[2 * dn], pf, vf[0], vf[1]);
                    mma_bf16(o[2 * dn + 1], pf, vf[2], vf[3]);
                }
            }
        }
        __syncthreads();
    }

#pragma unroll
    for (int i = 0; i < 2; ++i) {
        lrow[i] += __shfl_xor_sync(0xffffffffu, lrow[i], 1);
        lrow[i] += __shfl_xor_sync(0xffffffffu, lrow[i], 2);
        if (!valid[i]) continue;
        if (p.n_splits > 1) {
            float* dst = p.part + (((size_t)blockIdx.z * p.n_tokens + tok[i]) * p.heads + head[i]) * (DV + 2);
#pragma unroll
            for (int nt = 0; nt < 2 * ND; ++nt) {
                const int col = col0 + nt * 8 + 2 * tq;
                if (col < DV) *reinterpret_cast<float2*>(dst + col) = make_float2(o[nt][2 * i], o[nt][2 * i + 1]);
            }
            if (side == 0 && tq == 0) {
                dst[DV] = mrow[i];
                dst[DV + 1] = lrow[i];
            }
            continue;
        }
        const float inv = lrow[i] > 0.f ? 1.f / lrow[i] : 0.f;
        __nv_bfloat16* op = p.out + (size_t)tok[i] * p.out_stride + p.out_col + (size_t)head[i] * DV;
#pragma unroll
        for (int nt = 0; nt < 2 * ND; ++nt) {
            const int col = col0 + nt * 8 + 2 * tq;
            if (col < DV) *reinterpret_cast<uint32_t*>(op + col) = pack_bf16(o[nt][2 * i] * inv, o[nt][2 * i + 1] * inv);
        }
    }
}

// The runs of a sequence's keys meet: out = sum_s o_s 2^(m_s - m) / sum_s l_s 2^(m_s - m), m the largest maximum of the
// runs that saw a key (or hold the sink), in the order of the runs.  A CTA a (token, head).
__global__ void __launch_bounds__(128)
attention_latent_merge_kernel(const float* __restrict__ part, int n_splits, int n_tokens, int heads, int DV, const int* __restrict__ cu_q,
                              __nv_bfloat16* __restrict__ out, int out_stride, int out_col) {
    pdl_launch();
    pdl_wait();
    const int t = blockIdx.x, h = blockIdx.y;
    if (cu_q[t + 1] - cu_q[t] <= 0) return;            // a padding token: its row was cleared
    const size_t stride = (size_t)n_tokens * heads * (DV + 2);
    const float* src = part + ((size_t)t * heads + h) * (DV + 2);
    float w[16];
    float m = -INFINITY, l = 0.f;
    for (int s = 0; s < n_splits; ++s)
        if (src[s * stride + DV + 1] > 0.f) m = fmaxf(m, src[s * stride + DV]);
    for (int s = 0; s < n_splits; ++s) {
        const float ls = src[s * stride + DV + 1];
        w[s] = ls > 0.f ? fast_exp2(src[s * stride + DV] - m) : 0.f;
        l += ls * w[s];
    }
    const float inv = l > 0.f ? 1.f / l : 0.f;
    for (int c = threadIdx.x; c < DV; c += 128) {
        float acc = 0.f;
        for (int s = 0; s < n_splits; ++s)
            if (w[s] > 0.f) acc = fmaf(src[s * stride + c], w[s], acc);
        out[(size_t)t * out_stride + out_col + (size_t)h * DV + c] = __float2bfloat16_rn(acc * inv);
    }
}

template <int DVT, int KBL, int MINB = 1, int WPS = 2>
cudaError_t launch_latent_as(const LatentParams& p, int n_tiles, int head_groups, cudaStream_t stream) {
    static std::atomic<unsigned long long> done{0};
    const int bytes = (LAT_ROWS + 2 * KBL) * (p.D + 8) * 2 + 4 * WPS * (KBL / 8) * 32 * 16;
    cudaError_t e = allow_dynamic_smem(attention_latent_kernel<DVT, KBL, MINB, WPS>, 200 * 1024, done);
    if (e != cudaSuccess) return e;
    e = launch(attention_latent_kernel<DVT, KBL, MINB, WPS>, dim3(n_tiles, head_groups, p.n_splits), dim3(128 * WPS), bytes, stream, p);
    if (e != cudaSuccess || p.n_splits <= 1) return e;
    return launch(attention_latent_merge_kernel, dim3(n_tiles, p.heads), dim3(128), 0, stream, (const float*)p.part, p.n_splits, p.n_tokens,
                  p.heads, p.DV, p.cu_q, p.out, p.out_stride, p.out_col);
}

}  // namespace

int attention_latent_tile_rows() { return LAT_ROWS; }

// rows of ``key`` numbers whose first ``v_dim`` are the value: both multiples of 16, values of up to 512 numbers, and a
// tile's queries with two blocks of keys within the shared memory
bool attention_latent_supports(int key, int v_dim) {
    if (key % 16 || v_dim % 16 || v_dim < 16 || v_dim > 512 || v_dim > key) return false;
    const int kbl = 32;
    const int warps = v_dim > 256 ? 16 : 8;
    return (LAT_ROWS + 2 * kbl) * (key + 8) * 2 + warps * (kbl / 8) * 32 * 16 <= 200 * 1024;
}

cudaError_t launch_attention_latent(const void* q, int q_stride, int q_col, void* out, int out_stride, int out_col, const void* pages,
                                    const int* cu_q, const int* q_start, const int* block_table, int table_stride, const int* tiles,
                                    int n_tiles, int n_pages, int heads, int key, int v_dim, int page_size, float scale,
                                    const float* sinks, int n_splits, float* part, int n_tokens, cudaStream_t stream) {
    if (n_tiles == 0) return cudaSuccess;
    if (!attention_latent_supports(key, v_dim)) return cudaErrorInvalidValue;
    if (n_splits < 1 || n_splits > 16 || (n_splits > 1 && (tiles != nullptr || part == nullptr))) return cudaErrorInvalidValue;
    const int hpt = heads < LAT_ROWS ? heads : LAT_ROWS;
    LatentParams p = {(const __nv_bfloat16*)q, q_stride, q_col, (__nv_bfloat16*)out, out_stride, out_col, (const __nv_bfloat16*)pages,
                      cu_q, q_start, block_table, table_stride, reinterpret_cast<const int2*>(tiles), n_pages, heads, page_size, key,
                      v_dim, scale * 1.4426950408889634f, sinks, LAT_ROWS / hpt, hpt, n_splits, n_tokens, part};
    const int groups = (heads + hpt - 1) / hpt;
    if (v_dim <= 64) return launch_latent_as<64, 32, 2>(p, n_tiles, groups, stream);
    if (v_dim <= 128) return launch_latent_as<128, 32, 2>(p, n_tiles, groups, stream);
    if (v_dim <= 256) return launch_latent_as<256, 32, 2>(p, n_tiles, groups, stream);
    // wider values: one CTA an SM.  A step of single tokens runs four warps a slab (measured at rows of 576 numbers and 32
    // heads: 70 us against 79 us for 64 sequences of 1,024 keys); prompt portions two (3.50 ms against 3.61 ms for 4,096 tokens)
    if (p.tiles == nullptr) return launch_latent_as<512, 32, 1, 4>(p, n_tiles, groups, stream);
    return launch_latent_as<512, 32, 1, 2>(p, n_tiles, groups, stream);
}

}  // namespace vtb
