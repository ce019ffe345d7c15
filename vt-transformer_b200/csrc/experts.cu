// Mixture of experts: the routing step between the two packed products.
//
// The experts' gate and up matrices are one packed matrix and their down matrices are packed along the inner dimension,
// so a token's feed-forward is two products over all experts; what makes it a mixture is this kernel between them.  One
// block a token: a warp picks the `top` largest router logits (32-bit; the lower index among equals), forms the softmax
// over the picked logits, and the block multiplies the picked experts' columns of the activation by their weights and
// clears the others', so that the second product adds up exactly the chosen experts' results.
//
// For long portions the picks are grouped instead: `route_topk` leaves each token's picks and weights, `expert_lists`
// the picks of every expert in rising order (one block an expert, no atomics: the order is fixed), `gather_picks` the
// input rows sorted by expert, and after the experts' products over their slices `combine_picks` adds a token's picks
// in the order of the picks, in 32-bit.
#include "common.cuh"
#include "kernels.h"
#include "launch.cuh"

namespace vtb {

namespace {
constexpr int kMaxExperts = 1024;
constexpr int kRouteThreads = 128;
}

// The `top` largest of z[0 .. experts) (the lower index among equals), by the first warp of the block: picked[k] and
// picked_z[k] in falling order; z is used up.  Then w[e] = the pick's weight (0 for the others) if w is given: mode 0 the
// softmax over the picked logits; mode 1 each pick's sigmoid(logit) over the picks' sum of them (+ 1e-20), times `scale`.
__device__ __forceinline__ void pick_top(float* z, float* w, int* picked, float* picked_z, int experts, int top, int mode = 0,
                                         float scale = 1.f) {
    const int lane = threadIdx.x & 31;
    if (threadIdx.x >= 32) return;
    for (int k = 0; k < top; ++k) {
        float best = -INFINITY;
        int at = 0x7fffffff;
        for (int e = lane; e < experts; e += 32) {
            const float v = z[e];
            if (at == 0x7fffffff || v > best) { best = v; at = e; }      // a lane meets its experts in rising order
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oa = __shfl_xor_sync(0xffffffffu, at, o);
            if (oa != 0x7fffffff && (at == 0x7fffffff || ov > best || (ov == best && oa < at))) { best = ov; at = oa; }
        }
        if (lane == 0) {
            picked[k] = at;
            picked_z[k] = best;
            z[at] = -INFINITY;
        }
        __syncwarp();
    }
    if (lane == 0 && mode == 1) {
        float sum = 0.f;
        for (int k = 0; k < top; ++k) {
            picked_z[k] = 1.f / (1.f + expf(-picked_z[k]));
            sum += picked_z[k];
        }
        for (int k = 0; k < top; ++k) {
            const float wk = picked_z[k] / (sum + 1e-20f) * scale;
            picked_z[k] = wk;
            if (w) w[picked[k]] = wk;
        }
    } else if (lane == 0) {
        const float mx = picked_z[0];                  // the first pick is the largest
        float sum = 0.f;
        for (int k = 0; k < top; ++k) sum += expf(picked_z[k] - mx);
        for (int k = 0; k < top; ++k) {
            const float wk = expf(picked_z[k] - mx) / sum;
            picked_z[k] = wk;                          // from here on: the pick's weight
            if (w) w[picked[k]] = wk;
        }
    }
}

// z[e] = logits[t, e], or, with the router's matrix [experts, width] (32-bit) and the token's input row x [width], the
// dot product formed here in 32-bit: a warp an expert, a lane the same columns of every expert, the lanes' sums added by
// the warp: the order depends on the width alone.
template <typename T>
__device__ __forceinline__ void router_logits(float* z, const float* __restrict__ logits, const T* __restrict__ x,
                                              const float* __restrict__ router, int width, int experts, int t) {
    if (x == nullptr) {
        for (int e = threadIdx.x; e < experts; e += blockDim.x) z[e] = logits[(size_t)t * experts + e];
        return;
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
    const T* xr = x + (size_t)t * width;
    for (int e = warp; e < experts; e += warps) {
        const float* rr = router + (size_t)e * width;
        float acc = 0.f;
        for (int c = lane * 8; c < width; c += 256) {
            float a[8], b[8];
            Vec8<T>::load(xr + c, a);
            Vec8<float>::load(rr + c, b);
#pragma unroll
            for (int j = 0; j < 8; ++j) acc = fmaf(a[j], b[j], acc);
        }
        acc = warp_sum(acc);
        if (lane == 0) z[e] = acc;
    }
}

template <typename T>
__global__ void __launch_bounds__(kRouteThreads)
route_experts_kernel(const float* __restrict__ logits, const T* __restrict__ x, const float* __restrict__ router, int width,
                     int experts, int top, T* __restrict__ act, int act_stride, int inter, int mode, float scale) {
    __shared__ float z[kMaxExperts];          // the logits; a picked one is taken out
    __shared__ float w[kMaxExperts];          // the experts' weights, zero for those not picked
    __shared__ float picked_z[kMaxExperts];
    __shared__ int picked[kMaxExperts];
    pdl_launch();
    pdl_wait();
    const int t = blockIdx.x;
    for (int e = threadIdx.x; e < experts; e += blockDim.x) w[e] = 0.f;
    router_logits(z, logits, x, router, width, experts, t);
    __syncthreads();
    pick_top(z, w, picked, picked_z, experts, top, mode, scale);
    __syncthreads();
    T* row = act + (size_t)t * act_stride;
    if (inter % 8 == 0 && act_stride % 8 == 0 && (reinterpret_cast<uintptr_t>(act) & 15) == 0) {
        const int per = inter / 8;
        for (int c = threadIdx.x; c < experts * per; c += blockDim.x) {
            const float we = w[c / per];
            float v[8];
            if (we > 0.f) {
                Vec8<T>::load(row + c * 8, v);
#pragma unroll
                for (int j = 0; j < 8; ++j) v[j] *= we;
            } else {
#pragma unroll
                for (int j = 0; j < 8; ++j) v[j] = 0.f;
            }
            Vec8<T>::store(row + c * 8, v);
        }
        return;
    }
    for (int c = threadIdx.x; c < experts * inter; c += blockDim.x) {
        const float we = w[c / inter];
        row[c] = from_float<T>(we > 0.f ? to_float(row[c]) * we : 0.f);
    }
}

// The picks themselves: ids[t, k] and weights[t, k] in falling order of the logits (for the grouped products).
template <typename T>
__global__ void __launch_bounds__(kRouteThreads)
route_topk_kernel(const float* __restrict__ logits, const T* __restrict__ x, const float* __restrict__ router, int width, int experts,
                  int top, int* __restrict__ ids, float* __restrict__ weights, int mode, float scale) {
    __shared__ float z[kMaxExperts];
    __shared__ float picked_z[kMaxExperts];
    __shared__ int picked[kMaxExperts];
    pdl_launch();
    pdl_wait();
    const int t = blockIdx.x;
    router_logits(z, logits, x, router, width, experts, t);
    __syncthreads();
    pick_top(z, nullptr, picked, picked_z, experts, top, mode, scale);
    __syncthreads();
    for (int k = threadIdx.x; k < top; k += blockDim.x) {
        ids[(size_t)t * top + k] = picked[k];
        weights[(size_t)t * top + k] = picked_z[k];
    }
}

// One block an expert: the picks (flat index t * top + k) that chose it, in rising order, into lists[e, 0 .. counts[e]).
__global__ void __launch_bounds__(256)
expert_lists_kernel(const int* __restrict__ ids, int n_picks, int list_stride, int* __restrict__ lists, int* __restrict__ counts) {
    __shared__ int warp_total[8];
    __shared__ int running;
    pdl_launch();
    pdl_wait();
    const int e = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (threadIdx.x == 0) running = 0;
    __syncthreads();
    for (int base = 0; base < n_picks; base += 256) {
        const int i = base + threadIdx.x;
        const bool mine = i < n_picks && ids[i] == e;
        const unsigned vote = __ballot_sync(0xffffffffu, mine);
        if (lane == 0) warp_total[warp] = __popc(vote);
        __syncthreads();
        int before = running;
        for (int w = 0; w < warp; ++w) before += warp_total[w];
        if (mine) lists[(size_t)e * list_stride + before + __popc(vote & ((1u << lane) - 1u))] = i;
        __syncthreads();
        if (threadIdx.x == 0) {
            int total = 0;
            for (int w = 0; w < 8; ++w) total += warp_total[w];
            running += total;
        }
        __syncthreads();
    }
    if (threadIdx.x == 0) counts[e] = running;
}

// Row r of the sorted rows (expert by expert, each in the order of its list) is the input row of its pick's token;
// where[pick] = r tells the combining kernel where the pick's result lies.
template <typename T>
__global__ void __launch_bounds__(128)
gather_picks_kernel(const T* __restrict__ x, int width, const int* __restrict__ lists, int list_stride, const int* __restrict__ counts,
                    int experts, int top, T* __restrict__ sorted, int* __restrict__ where) {
    __shared__ int src;
    pdl_launch();
    pdl_wait();
    const int r = blockIdx.x;
    if (threadIdx.x == 0) {
        int e = 0, off = 0;
        while (e < experts && off + counts[e] <= r) off += counts[e++];
        src = e < experts ? lists[(size_t)e * list_stride + (r - off)] : -1;
        if (src >= 0) where[src] = r;
    }
    __syncthreads();
    if (src < 0) return;
    const T* from = x + (size_t)(src / top) * width;
    T* to = sorted + (size_t)r * width;
    for (int c = threadIdx.x * 8; c < width; c += blockDim.x * 8) {
        float v[8];
        Vec8<T>::load(from + c, v);
        Vec8<T>::store(to + c, v);
    }
}

// out[t] = sum_k weights[t, k] * y[where[t * top + k]] (+ shared[t]) in 32-bit, in the order of k, one rounding.
template <typename T>
__global__ void __launch_bounds__(128)
combine_picks_kernel(const T* __restrict__ y, int width, const int* __restrict__ where, const float* __restrict__ weights, int top,
                     const T* __restrict__ shared_y, T* __restrict__ out) {
    pdl_launch();
    pdl_wait();
    const int t = blockIdx.x;
    for (int c = threadIdx.x * 8; c < width; c += blockDim.x * 8) {
        float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        for (int k = 0; k < top; ++k) {
            const float wk = weights[(size_t)t * top + k];
            float v[8];
            Vec8<T>::load(y + (size_t)where[(size_t)t * top + k] * width + c, v);
#pragma unroll
            for (int j = 0; j < 8; ++j) acc[j] = fmaf(wk, v[j], acc[j]);
        }
        if (shared_y != nullptr) {
            float v[8];
            Vec8<T>::load(shared_y + (size_t)t * width + c, v);
#pragma unroll
            for (int j = 0; j < 8; ++j) acc[j] += v[j];
        }
        Vec8<T>::store(out + (size_t)t * width + c, acc);
    }
}

cudaError_t launch_route_topk(int x_dtype, const float* logits, const void* x, const float* router, int width, int n_tokens, int experts,
                              int top, int* ids, float* weights, cudaStream_t stream, int mode, float scale) {
    if (n_tokens == 0) return cudaSuccess;
    if (experts < 1 || experts > kMaxExperts || top < 1 || top > experts || (x != nullptr && width % 8)) return cudaErrorInvalidValue;
    if (x_dtype == kBF16)
        return launch(route_topk_kernel<__nv_bfloat16>, n_tokens, kRouteThreads, 0, stream, logits, (const __nv_bfloat16*)x, router, width,
                      experts, top, ids, weights, mode, scale);
    return launch(route_topk_kernel<float>, n_tokens, kRouteThreads, 0, stream, logits, (const float*)x, router, width, experts, top, ids,
                  weights, mode, scale);
}

cudaError_t launch_expert_lists(const int* ids, int n_picks, int experts, int list_stride, int* lists, int* counts, cudaStream_t stream) {
    if (experts == 0) return cudaSuccess;
    return launch(expert_lists_kernel, experts, 256, 0, stream, ids, n_picks, list_stride, lists, counts);
}

cudaError_t launch_gather_picks(int dtype, const void* x, int width, const int* lists, int list_stride, const int* counts, int experts,
                                int top, int n_picks, void* sorted, int* where, cudaStream_t stream) {
    if (n_picks == 0) return cudaSuccess;
    if (width % 8) return cudaErrorInvalidValue;
    if (dtype == kBF16)
        return launch(gather_picks_kernel<__nv_bfloat16>, n_picks, 128, 0, stream, (const __nv_bfloat16*)x, width, lists, list_stride,
                      counts, experts, top, (__nv_bfloat16*)sorted, where);
    return launch(gather_picks_kernel<float>, n_picks, 128, 0, stream, (const float*)x, width, lists, list_stride, counts, experts, top,
                  (float*)sorted, where);
}

cudaError_t launch_combine_picks(int dtype, const void* y, int width, const int* where, const float* weights, int top, int n_tokens,
                                 const void* shared_y, void* out, cudaStream_t stream) {
    if (n_tokens == 0) return cudaSuccess;
    if (width % 8) return cudaErrorInvalidValue;
    if (dtype == kBF16)
        return launch(combine_picks_kernel<__nv_bfloat16>, n_tokens, 128, 0, stream, (const __nv_bfloat16*)y, width, where, weights, top,
                      (const __nv_bfloat16*)shared_y, (__nv_bfloat16*)out);
    return launch(combine_picks_kernel<float>, n_tokens, 128, 0, stream, (const float*)y, width, where, weights, top,
                  (const float*)shared_y, (float*)out);
}

cudaError_t launch_route_experts(int dtype, const float* logits, const void* x, const float* router, int width, int n_tokens, int experts,
                                 int top, void* act, int act_stride, int inter, cudaStream_t stream, int mode, float scale) {
    if (n_tokens == 0) return cudaSuccess;
    if (experts < 1 || experts > kMaxExperts || top < 1 || top > experts || (x != nullptr && width % 8)) return cudaErrorInvalidValue;
    if (dtype == kBF16)
        return launch(route_experts_kernel<__nv_bfloat16>, n_tokens, kRouteThreads, 0, stream, logits, (const __nv_bfloat16*)x, router, width,
                      experts, top, (__nv_bfloat16*)act, act_stride, inter, mode, scale);
    return launch(route_experts_kernel<float>, n_tokens, kRouteThreads, 0, stream, logits, (const float*)x, router, width, experts, top,
                  (float*)act, act_stride, inter, mode, scale);
}

}  // namespace vtb
