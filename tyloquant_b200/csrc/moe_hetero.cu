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
};

constexpr bool hetero_has_codec(int bits, int t8) {
    return (bits == 2 && t8 == 2) || (bits == 3 && t8 == 3) || (bits == 4 && t8 == 3) || (bits == 5 && t8 == 4) || (bits == 6 && t8 == 3) ||
           (bits == 8 && t8 == 3) || (bits == 8 && t8 == 6);
}

__global__ void __launch_bounds__(256, 2) moe_hetero_gemv1_kernel(const __grid_constant__ HeteroArgs h) {
    extern __shared__ __align__(16) unsigned char smem[];
    pdl_wait_b();   // the routing table comes from the previous kernel
    const int e = h.base.route_ids[blockIdx.y];
    if (e < 0) return;
    const int pool = h.base.expert_pool[e];
    if (pool < 0) return;
    GemvArgsB a = h.base;
    a.pool = pool;
    const NintDevB& w = h.pools[pool];
    switch (w.bits * 16 + w.t8) {
        case 2 * 16 + 2: gemv1_bl_body<NintCodec<2, 2>>(a, w, smem); break;
        case 3 * 16 + 3: gemv1_bl_body<NintCodec<3, 3>>(a, w, smem); break;
        case 4 * 16 + 3: gemv1_bl_body<NintCodec<4, 3>>(a, w, smem); break;
        case 5 * 16 + 4: gemv1_bl_body<NintCodec<5, 4>>(a, w, smem); break;
        case 6 * 16 + 3: gemv1_bl_body<NintCodec<6, 3>>(a, w, smem); break;
        case 8 * 16 + 3: gemv1_bl_body<NintCodec<8, 3>>(a, w, smem); break;
        case 8 * 16 + 6: gemv1_bl_body<NintCodec<8, 6>>(a, w, smem); break;
        default: break;
    }
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
    const int want = (2 * device_sm_count(device) + pairs - 1) / std::max(pairs, 1);
    const int splits = std::max(1, std::min(base.rb_per_expert, want));
    base.rb_per_cta = (base.rb_per_expert + splits - 1) / splits;
    base.private_sums = base.rb_per_cta <= 8;
    h.base = base;
    const size_t smem = (size_t)((base.private_sums ? 8 : 1) + 1) * base.rb_per_cta * 16 * 4 + ring;
    static bool attr_set[64] = {false};
    if (smem > 48 * 1024 && !attr_set[device]) {
        MFQB_CUDA(cudaFuncSetAttribute(moe_hetero_gemv1_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        attr_set[device] = true;
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
    MFQB_CUDA(cudaLaunchKernelEx(&cfg, moe_hetero_gemv1_kernel, h));
    return true;
}

}  // namespace mfqb
