// Mixture-of-experts routing and pointwise glue: top-k router, deterministic route plan,
// SwiGLU split, weighted reduce.
#include <cuda_bf16.h>

#include <algorithm>
#include <cfloat>
#include <climits>

#include "cuda_util.h"

namespace mfqb {

// ---- top-k router: one warp per token ---------------------------------------------------
// Selection is exact: score comparisons only, ties to the smaller expert id, NaN -> -FLT_MAX
// (mfq/kernels/cuda/moe.cu:124-263).
__device__ __forceinline__ bool score_before(float sa, int ea, float sb, int eb) { return sa > sb || (sa == sb && ea < eb); }

__global__ void __launch_bounds__(128) moe_topk_kernel(const float* __restrict__ logits, const float* __restrict__ bias,
                                                        int32_t* __restrict__ ids, float* __restrict__ weights, int tokens,
                                                        int experts, int k, int mode, int normalize, float norm_floor,
                                                        float scale) {
    const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (row >= tokens) return;
    const float* z = logits + (size_t)row * experts;
    auto clean = [](float v) { return isnan(v) ? -FLT_MAX : v; };
    float smax = 0.f, ssum = 1.f;
    if (mode == MFQB_ROUTER_SOFTMAX) {
        smax = -INFINITY;
        for (int e = lane; e < experts; e += 32) smax = fmaxf(smax, clean(z[e]));
        for (int o = 16; o; o >>= 1) smax = fmaxf(smax, __shfl_xor_sync(0xffffffffu, smax, o));
        ssum = 0.f;
        for (int e = lane; e < experts; e += 32) ssum += expf(clean(z[e]) - smax);
        for (int o = 16; o; o >>= 1) ssum += __shfl_xor_sync(0xffffffffu, ssum, o);
    }
    auto weight_of = [&](float raw) {
        if (mode == MFQB_ROUTER_DELAYED_SOFTMAX) return raw;
        if (mode == MFQB_ROUTER_SIGMOID) return 1.0f / (1.0f + expf(-raw));
        if (mode == MFQB_ROUTER_SQRT_SOFTPLUS) return sqrtf(raw > 20.0f ? raw : log1pf(expf(raw)));
        return expf(raw - smax) / ssum;
    };
    int chosen[16];
    float my_weight = 0.f;   // lane r keeps the weight of rank r
    for (int r = 0; r < k; ++r) {
        float bs = -INFINITY, bw = -INFINITY;
        int be = INT_MAX;
        for (int e = lane; e < experts; e += 32) {
            bool taken = false;
            for (int p = 0; p < r; ++p) taken |= chosen[p] == e;
            if (taken) continue;
            const float wgt = weight_of(clean(z[e]));
            const float sc = wgt + (bias ? bias[e] : 0.0f);
            if (score_before(sc, e, bs, be)) { bs = sc; bw = wgt; be = e; }
        }
        for (int o = 16; o; o >>= 1) {
            const float os = __shfl_xor_sync(0xffffffffu, bs, o), ow = __shfl_xor_sync(0xffffffffu, bw, o);
            const int oe = __shfl_xor_sync(0xffffffffu, be, o);
            if (score_before(os, oe, bs, be)) { bs = os; bw = ow; be = oe; }
        }
        chosen[r] = be;
        if (lane == r) my_weight = bw;
        if (lane == 0) ids[(size_t)row * k + r] = be;
    }
    float v = lane < k ? my_weight : 0.f;
    if (mode == MFQB_ROUTER_DELAYED_SOFTMAX) {
        float m = lane < k ? v : -INFINITY;
        for (int o = 16; o; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
        v = lane < k ? expf(v - m) : 0.f;
        float d = v;
        for (int o = 16; o; o >>= 1) d += __shfl_xor_sync(0xffffffffu, d, o);
        v /= d;
    } else if (normalize) {
        float d = v;
        for (int o = 16; o; o >>= 1) d += __shfl_xor_sync(0xffffffffu, d, o);
        v /= fmaxf(d, norm_floor);
    }
    if (lane < k) weights[(size_t)row * k + lane] = v * scale;
}

// The same selection for up to 32 * EPL experts: a lane keeps its experts' weights and scores in
// registers (computed once), and a bit per expert marks the ones already chosen.  Same operations in
// the same order as moe_topk_kernel, so both give identical ids and weights.
template <int EPL>
__global__ void __launch_bounds__(128) moe_topk_regs_kernel(const float* __restrict__ logits, const float* __restrict__ bias,
                                                             int32_t* __restrict__ ids, float* __restrict__ weights, int tokens,
                                                             int experts, int k, int mode, int normalize, float norm_floor,
                                                             float scale) {
    const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (row >= tokens) return;
    const float* z = logits + (size_t)row * experts;
    float raw[EPL], bs_add[EPL];
    unsigned taken = 0u;   // bit j: expert lane + 32 j is out of range or already chosen
#pragma unroll
    for (int j = 0; j < EPL; ++j) {
        const int e = lane + 32 * j;
        const bool ok = e < experts;
        const float v = ok ? z[e] : 0.f;
        raw[j] = isnan(v) ? -FLT_MAX : v;
        bs_add[j] = (ok && bias) ? bias[e] : 0.f;
        if (!ok) taken |= 1u << j;
    }
    float smax = 0.f, ssum = 1.f;
    if (mode == MFQB_ROUTER_SOFTMAX) {
        smax = -INFINITY;
#pragma unroll
        for (int j = 0; j < EPL; ++j)
            if (!((taken >> j) & 1u)) smax = fmaxf(smax, raw[j]);
        for (int o = 16; o; o >>= 1) smax = fmaxf(smax, __shfl_xor_sync(0xffffffffu, smax, o));
        ssum = 0.f;
#pragma unroll
        for (int j = 0; j < EPL; ++j)
            if (!((taken >> j) & 1u)) ssum += expf(raw[j] - smax);
        for (int o = 16; o; o >>= 1) ssum += __shfl_xor_sync(0xffffffffu, ssum, o);
    }
    float wg[EPL], sc[EPL];
#pragma unroll
    for (int j = 0; j < EPL; ++j) {
        float wv;
        if (mode == MFQB_ROUTER_DELAYED_SOFTMAX) wv = raw[j];
        else if (mode == MFQB_ROUTER_SIGMOID) wv = 1.0f / (1.0f + expf(-raw[j]));
        else if (mode == MFQB_ROUTER_SQRT_SOFTPLUS) wv = sqrtf(raw[j] > 20.0f ? raw[j] : log1pf(expf(raw[j])));
        else wv = expf(raw[j] - smax) / ssum;
        wg[j] = wv;
        sc[j] = wv + bs_add[j];
    }
    float my_weight = 0.f;   // lane r keeps the weight of rank r
    for (int r = 0; r < k; ++r) {
        float bs = -INFINITY, bw = -INFINITY;
        int be = INT_MAX;
#pragma unroll
        for (int j = 0; j < EPL; ++j)
            if (!((taken >> j) & 1u) && score_before(sc[j], lane + 32 * j, bs, be)) { bs = sc[j]; bw = wg[j]; be = lane + 32 * j; }
        for (int o = 16; o; o >>= 1) {
            const float os = __shfl_xor_sync(0xffffffffu, bs, o), ow = __shfl_xor_sync(0xffffffffu, bw, o);
            const int oe = __shfl_xor_sync(0xffffffffu, be, o);
            if (score_before(os, oe, bs, be)) { bs = os; bw = ow; be = oe; }
        }
        if (lane == (be & 31)) taken |= 1u << (be >> 5);
        if (lane == r) my_weight = bw;
        if (lane == 0) ids[(size_t)row * k + r] = be;
    }
    float v = lane < k ? my_weight : 0.f;
    if (mode == MFQB_ROUTER_DELAYED_SOFTMAX) {
        float m = lane < k ? v : -INFINITY;
        for (int o = 16; o; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
        v = lane < k ? expf(v - m) : 0.f;
        float d = v;
        for (int o = 16; o; o >>= 1) d += __shfl_xor_sync(0xffffffffu, d, o);
        v /= d;
    } else if (normalize) {
        float d = v;
        for (int o = 16; o; o >>= 1) d += __shfl_xor_sync(0xffffffffu, d, o);
        v /= fmaxf(d, norm_floor);
    }
    if (lane < k) weights[(size_t)row * k + lane] = v * scale;
}

// ---- route plan ------------------------------------------------------------------------------
// counts -> exclusive scan -> stable placement (one warp per expert walks the pairs in order),
// so every expert's segment lists its pairs in ascending order: the plan is deterministic.
__global__ void route_count_kernel(const int32_t* __restrict__ ids, int pairs, int experts, int32_t* __restrict__ counts) {
    const int e = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (e >= experts) return;
    int n = 0;
    for (int p = lane; p < pairs; p += 32) n += ids[p] == e;
    for (int o = 16; o; o >>= 1) n += __shfl_xor_sync(0xffffffffu, n, o);
    if (lane == 0) counts[e] = n;
}

__global__ void route_scan_kernel(int experts, int tile_m, int32_t* __restrict__ expert_bounds, int32_t* __restrict__ tile_bounds) {
    // expert_bounds[1..E] holds the counts on entry; one thread scans (E <= 4096, a few microseconds
    // at most, off the critical path of the expert matmuls of small batches which do not use the plan)
    if (threadIdx.x == 0 && blockIdx.x == 0) {
        int run = 0, tiles = 0;
        expert_bounds[0] = 0;
        tile_bounds[0] = 0;
        for (int e = 0; e < experts; ++e) {
            const int c = expert_bounds[e + 1];
            run += c;
            tiles += (c + tile_m - 1) / tile_m;
            expert_bounds[e + 1] = run;
            tile_bounds[e + 1] = tiles;
        }
    }
}

__global__ void route_place_kernel(const int32_t* __restrict__ ids, int pairs, int experts,
                                   const int32_t* __restrict__ expert_bounds, int32_t* __restrict__ pair_order) {
    const int e = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (e >= experts) return;
    int at = expert_bounds[e];
    for (int base = 0; base < pairs; base += 32) {
        const int p = base + lane;
        const bool hit = p < pairs && ids[p] == e;
        const unsigned m = __ballot_sync(0xffffffffu, hit);
        if (hit) pair_order[at + __popc(m & ((1u << lane) - 1u))] = p;
        at += __popc(m);
    }
}

// The same plan in one launch for decode-sized batches: one CTA counts with shared-memory
// atomics, scans, and places (a warp per expert walks the pairs in order, as above).
constexpr int kRoutePlanSmallExperts = 1024, kRoutePlanSmallPairs = 4096;
__global__ void __launch_bounds__(1024) route_plan_small_kernel(const int32_t* __restrict__ ids, int pairs, int experts, int tile_m,
                                                                int32_t* __restrict__ expert_bounds, int32_t* __restrict__ tile_bounds,
                                                                int32_t* __restrict__ pair_order) {
    __shared__ int bounds[kRoutePlanSmallExperts + 1];
    __shared__ int ids_s[kRoutePlanSmallPairs];   // the placement below walks the ids once per expert: from shared memory
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarps = blockDim.x >> 5;
    for (int e = tid; e <= experts; e += blockDim.x) bounds[e] = 0;
    __syncthreads();
    for (int p = tid; p < pairs; p += blockDim.x) {
        const int e = ids[p];
        ids_s[p] = e;
        if (e >= 0 && e < experts) atomicAdd(&bounds[e + 1], 1);
    }
    __syncthreads();
    if (tid == 0) {
        int run = 0, tiles = 0;
        expert_bounds[0] = 0;
        tile_bounds[0] = 0;
        for (int e = 0; e < experts; ++e) {
            const int c = bounds[e + 1];
            bounds[e] = run;   // start of expert e's segment
            run += c;
            tiles += (c + tile_m - 1) / tile_m;
            expert_bounds[e + 1] = run;
            tile_bounds[e + 1] = tiles;
        }
    }
    __syncthreads();
    for (int e = warp; e < experts; e += nwarps) {
        int at = bounds[e];
        for (int base = 0; base < pairs; base += 32) {
            const int p = base + lane;
            const bool hit = p < pairs && ids_s[p] == e;
            const unsigned m = __ballot_sync(0xffffffffu, hit);
            if (hit) pair_order[at + __popc(m & ((1u << lane) - 1u))] = p;
            at += __popc(m);
        }
    }
}

// ---- pointwise glue -----------------------------------------------------------------------------
template <typename T>
__device__ __forceinline__ float to_f32(T v);
template <>
__device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T, typename O>
__global__ void swiglu_kernel(const T* __restrict__ gate_up, int rows, int f, O* __restrict__ hidden) {
    const size_t total = (size_t)rows * f;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const size_t r = i / f, j = i % f;
        const float g = to_f32(gate_up[r * 2 * f + j]), u = to_f32(gate_up[r * 2 * f + f + j]);
        const float v = u * g / (1.0f + expf(-g));
        if constexpr (sizeof(O) == 4) hidden[i] = v;
        else hidden[i] = __float2bfloat16_rn(v);
    }
}

template <typename T, typename O>
__global__ void weighted_reduce_kernel(const T* __restrict__ src, const float* __restrict__ weights, int tokens, int routes, int h,
                                       O* __restrict__ y) {
    const size_t total = (size_t)tokens * h;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const size_t t = i / h, j = i % h;
        float acc = 0.f;
        for (int r = 0; r < routes; ++r) acc += weights[t * routes + r] * to_f32(src[(t * routes + r) * h + j]);
        if constexpr (sizeof(O) == 4) y[i] = acc;
        else y[i] = __float2bfloat16_rn(acc);
    }
}

void launch_swiglu(const void* gate_up, int in_dtype, int rows, int f, void* hidden, cudaStream_t s) {
    const size_t total = (size_t)rows * f;
    if (total == 0) return;
    const int block = 256, grid = (int)std::min<size_t>((total + block - 1) / block, 148 * 8);
    if (in_dtype == MFQB_F32) swiglu_kernel<float, __nv_bfloat16><<<grid, block, 0, s>>>(static_cast<const float*>(gate_up), rows, f, static_cast<__nv_bfloat16*>(hidden));
    else swiglu_kernel<__nv_bfloat16, __nv_bfloat16><<<grid, block, 0, s>>>(static_cast<const __nv_bfloat16*>(gate_up), rows, f, static_cast<__nv_bfloat16*>(hidden));
    MFQB_CUDA(cudaGetLastError());
}

// float32 gate|up -> float32 activation (the library's own intermediate: no rounding between the two expert matmuls)
void launch_swiglu_f32(const float* gate_up, int rows, int f, float* hidden, cudaStream_t s) {
    const size_t total = (size_t)rows * f;
    if (total == 0) return;
    const int block = 256, grid = (int)std::min<size_t>((total + block - 1) / block, 148 * 8);
    swiglu_kernel<float, float><<<grid, block, 0, s>>>(gate_up, rows, f, hidden);
    MFQB_CUDA(cudaGetLastError());
}

void launch_weighted_reduce(const void* src, int in_dtype, const float* weights, int tokens, int routes, int h, void* y, int y_dtype,
                            cudaStream_t s) {
    const size_t total = (size_t)tokens * h;
    if (total == 0) return;
    const int block = 256, grid = (int)std::min<size_t>((total + block - 1) / block, 148 * 8);
    if (in_dtype == MFQB_F32) {
        if (y_dtype == MFQB_F32) weighted_reduce_kernel<float, float><<<grid, block, 0, s>>>(static_cast<const float*>(src), weights, tokens, routes, h, static_cast<float*>(y));
        else weighted_reduce_kernel<float, __nv_bfloat16><<<grid, block, 0, s>>>(static_cast<const float*>(src), weights, tokens, routes, h, static_cast<__nv_bfloat16*>(y));
    } else {
        if (y_dtype == MFQB_F32) weighted_reduce_kernel<__nv_bfloat16, float><<<grid, block, 0, s>>>(static_cast<const __nv_bfloat16*>(src), weights, tokens, routes, h, static_cast<float*>(y));
        else weighted_reduce_kernel<__nv_bfloat16, __nv_bfloat16><<<grid, block, 0, s>>>(static_cast<const __nv_bfloat16*>(src), weights, tokens, routes, h, static_cast<__nv_bfloat16*>(y));
    }
    MFQB_CUDA(cudaGetLastError());
}

void launch_route_plan(const int32_t* ids, int pairs, int experts, int tile_m, int32_t* expert_bounds, int32_t* tile_bounds,
                       int32_t* pair_order, cudaStream_t stream) {
    if (experts <= kRoutePlanSmallExperts && pairs <= kRoutePlanSmallPairs) {
        route_plan_small_kernel<<<1, 1024, 0, stream>>>(ids, pairs, experts, tile_m, expert_bounds, tile_bounds, pair_order);
        MFQB_CUDA(cudaGetLastError());
        return;
    }
    const int blocks = (experts + 3) / 4;
    route_count_kernel<<<blocks, 128, 0, stream>>>(ids, pairs, experts, expert_bounds + 1);
    route_scan_kernel<<<1, 32, 0, stream>>>(experts, tile_m, expert_bounds, tile_bounds);
    route_place_kernel<<<blocks, 128, 0, stream>>>(ids, pairs, experts, expert_bounds, pair_order);
    MFQB_CUDA(cudaGetLastError());
}

}  // namespace mfqb

using namespace mfqb;

extern "C" {
#pragma GCC visibility push(default)

int mfqb_moe_topk(const float* logits, int tokens, int experts, int k, int mode, const float* bias, int normalize,
                  float norm_floor, float scale, int32_t* ids, float* weights, mfqb_stream_t stream) {
    return guarded([&] {
        if (!logits || !ids || !weights) fail(MFQB_ERR_ARG, "mfqb_moe_topk: null argument");
        if (tokens < 0 || experts < 1 || experts > 4096) fail(MFQB_ERR_ARG, "mfqb_moe_topk: experts must be in [1, 4096]");
        if (k < 1 || k > 16 || k > experts) fail(MFQB_ERR_ARG, "mfqb_moe_topk: top_k must be in [1, min(16, experts)]");
        if (mode < 0 || mode > 3) fail(MFQB_ERR_ARG, "mfqb_moe_topk: unknown router mode %d", mode);
        if (tokens == 0) return;
        const dim3 grid((tokens + 3) / 4), block(128);
        if (experts <= 128) moe_topk_regs_kernel<4><<<grid, block, 0, stream>>>(logits, bias, ids, weights, tokens, experts, k, mode, normalize, norm_floor, scale);
        else if (experts <= 256) moe_topk_regs_kernel<8><<<grid, block, 0, stream>>>(logits, bias, ids, weights, tokens, experts, k, mode, normalize, norm_floor, scale);
        else if (experts <= 512) moe_topk_regs_kernel<16><<<grid, block, 0, stream>>>(logits, bias, ids, weights, tokens, experts, k, mode, normalize, norm_floor, scale);
        else moe_topk_kernel<<<grid, block, 0, stream>>>(logits, bias, ids, weights, tokens, experts, k, mode, normalize, norm_floor, scale);
        MFQB_CUDA(cudaGetLastError());
    });
}

int mfqb_moe_route_plan(const int32_t* ids, int tokens, int k, int experts, int tile_m, int32_t* expert_bounds,
                        int32_t* tile_bounds, int32_t* pair_order, mfqb_stream_t stream) {
    return guarded([&] {
        if (!ids || !expert_bounds || !tile_bounds || !pair_order) fail(MFQB_ERR_ARG, "mfqb_moe_route_plan: null argument");
        if (tokens < 0 || k < 1 || experts < 1 || tile_m < 1) fail(MFQB_ERR_ARG, "mfqb_moe_route_plan: bad sizes");
        launch_route_plan(ids, tokens * k, experts, tile_m, expert_bounds, tile_bounds, pair_order, stream);
    });
}

int mfqb_moe_swiglu(const void* gate_up, int in_dtype, int rows, int f, void* hidden_bf16, mfqb_stream_t stream) {
    return guarded([&] {
        if (!gate_up || !hidden_bf16 || rows < 0 || f < 1) fail(MFQB_ERR_ARG, "mfqb_moe_swiglu: bad argument");
        launch_swiglu(gate_up, in_dtype, rows, f, hidden_bf16, stream);
    });
}

int mfqb_moe_weighted_reduce(const void* expert_out, int in_dtype, const float* weights, int tokens, int routes, int h, void* y,
                             int y_dtype, mfqb_stream_t stream) {
    return guarded([&] {
        if (!expert_out || !weights || !y || tokens < 0 || routes < 1 || h < 1) fail(MFQB_ERR_ARG, "mfqb_moe_weighted_reduce: bad argument");
        launch_weighted_reduce(expert_out, in_dtype, weights, tokens, routes, h, y, y_dtype, stream);
    });
}

#pragma GCC visibility pop
}  // extern "C"
