// One launch for the routed single-row matmul over all precision cohorts of an NINTM record.
//
// At decode sizes a routed matmul is a handful of (token, route) pairs, and a launch per cohort
// costs more than the work.  This kernel takes every held cohort at once: a CTA looks up its
// pair's expert, the expert's cohort, and runs the single-row body of that cohort's codec.
// The codecs are those of the reference's per-expert precision profiles (mfq/kernels/cuda/moe.cu:35-41:
// (2,16) (3,24) (4,24) (5,28) (6,24) (8,24) (8,48)); records with other cohorts take one launch each.
// Replaces the heterogeneous single-launch path of the reference (cpp_runtime/mfq_decode.cpp:1093-1099, 3021-3023).
#include <algorithm>

#include "cuda_util.h"
#include "nint_gemv_bl_launch.cuh"

namespace mfqb {

constexpr int kHeteroMaxPools = 8;

struct HeteroArgs {
    GemvArgsB base;                      // routing tables, x, y, splits; base.w is unused
    NintDevB pools[kHeteroMaxPools];     // cohort tensors, indexed by expert_pool[e]
    const uint2* xq_g[kHeteroMaxPools];  // tile mode: quantised input planes of each cohort (by group size)
    const float2* gtab_g[kHeteroMaxPools];
};

constexpr bool hetero_has_codec(int bits, int t8) {
    return (bits == 2 && t8 == 2) || (bits == 3 && t8 == 3) || (bits == 4 && t8 == 3) || (bits == 5 && t8 == 4) || (bits == 6 && t8 == 3) ||
           (bits == 8 && t8 == 3) || (bits == 8 && t8 == 6);
}

template <int XMODE>
__global__ void __launch_bounds__(256, 2) moe_hetero_gemv1_kernel(const __grid_constant__ HeteroArgs h) {
    extern __shared__ __align__(16) unsigned char smem[];
    pdl_wait_b();   // the routing table comes from the previous kernel
    const int e = h.base.route_ids[blockIdx.y];
    // an id outside [0, n_experts) is ignored like a route to an expert that is not held here
    const int pool = (e >= 0 && e < h.base.n_experts) ? h.base.expert_pool[e] : -1;
    if (pool < 0) {
        if (h.base.route_w != nullptr) routed_absent_pair(h.base, blockIdx.y);
        return;
    }
    GemvArgsB a = h.base;
    a.pool = pool;
    const NintDevB& w = h.pools[pool];
    switch (w.bits * 16 + w.t8) {
        case 2 * 16 + 2: gemv1_bl_body<NintCodec<2, 2>, XMODE, false, true>(a, w, smem); break;
        case 3 * 16 + 3: gemv1_bl_body<NintCodec<3, 3>, XMODE, false, true>(a, w, smem); break;
        case 4 * 16 + 3: gemv1_bl_body<NintCodec<4, 3>, XMODE, false, true>(a, w, smem); break;
        case 5 * 16 + 4: gemv1_bl_body<NintCodec<5, 4>, XMODE, false, true>(a, w, smem); break;
        case 6 * 16 + 3: gemv1_bl_body<NintCodec<6, 3>, XMODE, false, true>(a, w, smem); break;
        case 8 * 16 + 3: gemv1_bl_body<NintCodec<8, 3>, XMODE, false, true>(a, w, smem); break;
        case 8 * 16 + 6: gemv1_bl_body<NintCodec<8, 6>, XMODE, false, true>(a, w, smem); break;
        default: break;
    }
}

// True when every held cohort has a codec in the all-cohort kernels.
bool moe_hetero_supported(const NintDevB* pools, const int* held, int npools) {
    if (npools > kHeteroMaxPools) return false;
    for (int i = 0; i < npools; ++i)
        if (held[i] && !hetero_has_codec(pools[i].bits, pools[i].t8)) return false;
    return true;
}

// Tile mode over all cohorts: blockIdx.y is a route-plan tile; the tile's expert selects the cohort.
template <int P>
__global__ void __launch_bounds__(256, 2) moe_hetero_tiles_kernel(const __grid_constant__ HeteroArgs h) {
    extern __shared__ __align__(16) unsigned char smem[];
    pdl_wait_b();   // route plan and quantised planes come from the previous kernels
    const int t = blockIdx.y, n_experts = h.base.n_experts;
    if (t >= h.base.tile_bounds[n_experts]) return;
    int lo = 0, hi = n_experts - 1;   // expert e with tile_bounds[e] <= t < tile_bounds[e + 1]
    while (lo < hi) {
        const int mid = (lo + hi + 1) >> 1;
        if (h.base.tile_bounds[mid] <= t) lo = mid;
        else hi = mid - 1;
    }
    const int pool = h.base.expert_pool[lo];
    if (pool < 0) return;
    GemvArgsB a = h.base;
    a.pool = pool;
    a.xq_g = h.xq_g[pool];
    a.gtab_g = h.gtab_g[pool];
    const NintDevB& w = h.pools[pool];
    switch (w.bits * 16 + w.t8) {
        case 2 * 16 + 2: gemvn_bl_body<NintCodec<2, 2>, P>(a, w, smem); break;
        case 3 * 16 + 3: gemvn_bl_body<NintCodec<3, 3>, P>(a, w, smem); break;
        case 4 * 16 + 3: gemvn_bl_body<NintCodec<4, 3>, P>(a, w, smem); break;
        case 5 * 16 + 4: gemvn_bl_body<NintCodec<5, 4>, P>(a, w, smem); break;
        case 6 * 16 + 3: gemvn_bl_body<NintCodec<6, 3>, P>(a, w, smem); break;
        case 8 * 16 + 3: gemvn_bl_body<NintCodec<8, 3>, P>(a, w, smem); break;
        case 8 * 16 + 6: gemvn_bl_body<NintCodec<8, 6>, P>(a, w, smem); break;
        default: break;
    }
}

// Launches the tile-mode matmul for all cohorts at once (tile_m = 2, 4 or 8 pairs per tile);
// xq / gtab: the quantised input planes to use for each cohort.  Returns false when a cohort has
// no codec here.
bool launch_moe_hetero_tiles(GemvArgsB base, const NintDevB* pools, const int* held, const uint2* const* xq, const float2* const* gtab,
                             int npools, int tile_m, int max_tiles, int device, cudaStream_t s) {
    // Tiles of eight pairs stay with one launch per cohort: there the work dwarfs the launches, and a
    // kernel holding every codec at four passes would need more registers than two CTAs per SM allow.
    if (tile_m > 4 || !moe_hetero_supported(pools, held, npools)) return false;
    HeteroArgs h{};
    const int passes = tile_m / 2;
    size_t dyn = 0;
    int t8max = 0;
    for (int i = 0; i < npools; ++i) {
        if (!held[i]) continue;
        h.pools[i] = pools[i];
        h.xq_g[i] = xq[i];
        h.gtab_g[i] = gtab[i];
        t8max = std::max(t8max, pools[i].t8);
    }
    base.m = tile_m;
    // most tiles of a launch sized by the upper bound are empty: split an expert's rows finely
    const int want = (2 * device_sm_count(device) + max_tiles - 1) / std::max(max_tiles, 1);
    const int splits = std::max(1, std::min(base.rb_per_expert, std::max(base.rb_per_expert / 8, want)));
    base.rb_per_cta = (base.rb_per_expert + splits - 1) / splits;
    for (int i = 0; i < npools; ++i)
        if (held[i])
            dyn = std::max(dyn, (size_t)(tile_m + 1) * base.rb_per_cta * 16 * 4 + (size_t)8 * 2 * tile_m * gemvn_bl_row_bytes(pools[i].t8) +
                                    (size_t)8 * gemvn_bl_stages(pools[i].rec_words, passes) * pools[i].rec_words * 4);
    if (dyn > 200 * 1024) return false;
    h.base = base;
    static bool attr_set[2][64] = {};   // per kernel (one or two passes) and device
    auto launch = [&](auto kernel) {
        bool& done = attr_set[passes - 1][device];
        if (!done) {
            MFQB_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
            done = true;
        }
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3((unsigned)splits, (unsigned)max_tiles);
        cfg.blockDim = dim3(256);
        cfg.dynamicSmemBytes = dyn;
        cfg.stream = s;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        const cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, h);
        if (e != cudaSuccess)
            fail(MFQB_ERR_CUDA, "all-cohort tile launch (grid %d x %d, %zu bytes of shared memory, tile of %d): %s", splits, max_tiles, dyn, tile_m,
                 cudaGetErrorString(e));
    };
    switch (passes) {
        case 1: launch(moe_hetero_tiles_kernel<1>); break;
        case 2: launch(moe_hetero_tiles_kernel<2>); break;
        default: return false;
    }
    return true;
}

// The same over the f16 batched kernel: tiles of 8 (NT = 1) or 16 (NT = 2) pairs, the input rows as scaled f16 in
// fragment order (base.x16f, base.x16f_tile_stride, base.x16_scale).
template <int NT>
__global__ void __launch_bounds__(256, 3) moe_hetero_tilesh_kernel(const __grid_constant__ HeteroArgs h) {
    extern __shared__ __align__(16) unsigned char smem[];
    pdl_wait_b();   // route plan and f16 rows come from the previous kernels
    const int t = blockIdx.y, n_experts = h.base.n_experts;
    if (t >= h.base.tile_bounds[n_experts]) return;
    int lo = 0, hi = n_experts - 1;   // expert e with tile_bounds[e] <= t < tile_bounds[e + 1]
    while (lo < hi) {
        const int mid = (lo + hi + 1) >> 1;
        if (h.base.tile_bounds[mid] <= t) lo = mid;
        else hi = mid - 1;
    }
    const int pool = h.base.expert_pool[lo];
    if (pool < 0) return;
    GemvArgsB a = h.base;
    a.pool = pool;
    const NintDevB& w = h.pools[pool];
    switch (w.bits * 16 + w.t8) {
        case 2 * 16 + 2: gemvh_bl_body<NintCodec<2, 2>, NT>(a, w, smem); break;
        case 3 * 16 + 3: gemvh_bl_body<NintCodec<3, 3>, NT>(a, w, smem); break;
        case 4 * 16 + 3: gemvh_bl_body<NintCodec<4, 3>, NT>(a, w, smem); break;
        case 5 * 16 + 4: gemvh_bl_body<NintCodec<5, 4>, NT>(a, w, smem); break;
        case 6 * 16 + 3: gemvh_bl_body<NintCodec<6, 3>, NT>(a, w, smem); break;
        case 8 * 16 + 3: gemvh_bl_body<NintCodec<8, 3>, NT>(a, w, smem); break;
        case 8 * 16 + 6: gemvh_bl_body<NintCodec<8, 6>, NT>(a, w, smem); break;
        default: break;
    }
}

// True when every held cohort can run on the f16 tile kernel (a codec here, group size in whole octets).
bool moe_hetero_tilesh_supported(const NintDevB* pools, const int* held, int npools) {
    if (!moe_hetero_supported(pools, held, npools)) return false;
    for (int i = 0; i < npools; ++i)
        if (held[i] && pools[i].gs != 8 * pools[i].t8) return false;
    return true;
}

// Launches the f16 tile-mode matmul for all cohorts at once (tile_m = 8 or 16 pairs per tile).
bool launch_moe_hetero_tilesh(GemvArgsB base, const NintDevB* pools, const int* held, int npools, int tile_m, int max_tiles, int device, cudaStream_t s) {
    if ((tile_m != 8 && tile_m != 16) || !moe_hetero_tilesh_supported(pools, held, npools)) return false;
    HeteroArgs h{};
    for (int i = 0; i < npools; ++i)
        if (held[i]) h.pools[i] = pools[i];
    base.m = tile_m;
    // most tiles of a launch sized by the upper bound are empty: split an expert's rows finely
    const int want = (2 * device_sm_count(device) + max_tiles - 1) / std::max(max_tiles, 1);
    const int splits = std::max(1, std::min(base.rb_per_expert, std::max(base.rb_per_expert / 8, want)));
    base.rb_per_cta = (base.rb_per_expert + splits - 1) / splits;
    size_t dyn = 0;
    for (int i = 0; i < npools; ++i)
        if (held[i])
            dyn = std::max(dyn, (size_t)(tile_m + 1) * base.rb_per_cta * 16 * 4 + (size_t)8 * gemvh_stages(pools[i].rec_words) * pools[i].rec_words * 4);
    if (dyn > 200 * 1024) return false;
    h.base = base;
    static bool attr_set[2][64] = {};   // per kernel (8 or 16 pairs) and device
    auto launch = [&](auto kernel, int which) {
        bool& done = attr_set[which][device];
        if (!done) {
            MFQB_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
            done = true;
        }
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3((unsigned)splits, (unsigned)max_tiles);
        cfg.blockDim = dim3(256);
        cfg.dynamicSmemBytes = dyn;
        cfg.stream = s;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        const cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, h);
        if (e != cudaSuccess)
            fail(MFQB_ERR_CUDA, "all-cohort f16 tile launch (grid %d x %d, %zu bytes of shared memory, tile of %d): %s", splits, max_tiles, dyn, tile_m,
                 cudaGetErrorString(e));
    };
    if (tile_m == 8) launch(moe_hetero_tilesh_kernel<1>, 0);
    else launch(moe_hetero_tilesh_kernel<2>, 1);
    return true;
}

// CTAs per pair (row splits) the all-cohort single-row launch uses for `pairs` pairs.
int moe_hetero_gemv1_splits(int rb_per_expert, int pairs, int device) {
    const int want = (2 * device_sm_count(device) + pairs - 1) / std::max(pairs, 1);
    return std::max(1, std::min(rb_per_expert, want));
}

// Launches the routed single-row matmul for all `npools` cohorts at once; returns false when a
// cohort has no codec in this kernel (the caller then launches cohort by cohort).
bool launch_moe_hetero_gemv1(GemvArgsB base, const NintDevB* pools, const int* held, int npools, int pairs, int device, cudaStream_t s) {
    if (npools > kHeteroMaxPools) return false;
    HeteroArgs h{};
    size_t ring = 0;
    for (int i = 0; i < npools; ++i) {
        if (!held[i]) continue;   // its experts map to pool -1 or are never routed here
        if (!hetero_has_codec(pools[i].bits, pools[i].t8)) return false;
        h.pools[i] = pools[i];
        ring = std::max(ring, (size_t)8 * gemv1_bl_stages(pools[i].rec_words) * pools[i].rec_words * 4);
    }
    base.m = 1;
    const int splits = moe_hetero_gemv1_splits(base.rb_per_expert, pairs, device);
    base.rb_per_cta = (base.rb_per_expert + splits - 1) / splits;
    base.private_sums = base.rb_per_cta <= 8;
    h.base = base;
    const size_t smem = (size_t)((base.private_sums ? 8 : 1) + 1) * base.rb_per_cta * 16 * 4 + ring;
    auto kernel = base.x_mode == 2 ? moe_hetero_gemv1_kernel<2> : (base.x_mode == 1 ? moe_hetero_gemv1_kernel<1> : moe_hetero_gemv1_kernel<0>);
    static bool attr_set[3][64] = {};
    if (smem > 48 * 1024 && !attr_set[base.x_mode][device]) {
        MFQB_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        attr_set[base.x_mode][device] = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)splits, (unsigned)pairs);
    cfg.blockDim = dim3(256);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    MFQB_CUDA(cudaLaunchKernelEx(&cfg, kernel, h));
    return true;
}

}  // namespace mfqb
