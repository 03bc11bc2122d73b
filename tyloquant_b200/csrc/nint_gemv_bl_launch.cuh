// Per-code-width launch tables of the byte-lane GEMV kernels; one translation unit per width
// (nint_gemv_bl_b*.cu) instantiates launch_gemv_bl_bits<BITS> so the widths compile in parallel.
#pragma once
#include "nint_gemvn_bl.cuh"
#include "nint_gemvh_bl.cuh"
#include "nint_gemvs.cuh"

namespace mfqb {

struct GemvPlanB {
    int grid = 1, grid_y = 1, threads = 256;
    const GemvMultiTable* multi = nullptr;   // the weights of a multi-weight launch (passes == -1)
    int* occupancy_out = nullptr;            // set: nothing is launched, the kernel's resident CTAs per SM for (threads, smem) are stored here
    int passes = 0;      // 0: single-row kernel; 1, 2, 4: batched kernel with that many two-row passes; -1: multi-weight single-row launch; -2: single-row kernel on a float32 gate|up row; -3: single-row kernel over (token, route) pairs of one cohort; -4: single-row kernel with the fused residual add + RMSNorm; 108, 116: f16 batched kernel for up to 8 or 16 rows
    size_t smem = 0;
};

template <int BITS>
cudaError_t launch_gemv_bl_bits(const GemvArgsB& a, const GemvPlanB& p, cudaStream_t stream);

// Streamed single-row kernel (nint_gemvs.cuh): grid = CTAs (one per SM), threads, dynamic shared memory.
struct GemvSPlan {
    int grid = 1, threads = 256;
    size_t smem = 0;
};
template <int BITS>
cudaError_t launch_gemvs_bits(const GemvSArgs& a, const GemvSPlan& p, cudaStream_t stream);

template <class C>
static cudaError_t launch_gemvs_codec(const GemvSArgs& a, const GemvSPlan& p, cudaStream_t stream) {
    auto kernel = gemvs_kernel<C>;
    // once per kernel and device: allow the largest dynamic shared memory any plan asks for
    static bool attr_set[64] = {};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev >= 0 && dev < 64 && !attr_set[dev]) {
        e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        if (e != cudaSuccess) return e;
        attr_set[dev] = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)p.grid);
    cfg.blockDim = dim3((unsigned)p.threads);
    cfg.dynamicSmemBytes = p.smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, a);
}

template <typename Kernel, typename... Extra>
static cudaError_t launch_kernel_pdl(Kernel kernel, const GemvArgsB& a, const GemvPlanB& p, cudaStream_t stream, const Extra&... extra) {
    if (p.smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)p.smem);
        if (e != cudaSuccess) return e;
    }
    if (p.occupancy_out) return cudaOccupancyMaxActiveBlocksPerMultiprocessor(p.occupancy_out, kernel, p.threads, p.smem);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)p.grid, (unsigned)p.grid_y);
    cfg.blockDim = dim3((unsigned)p.threads);
    cfg.dynamicSmemBytes = p.smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, a, extra...);
}

template <class C>
static cudaError_t launch_gemv_codec(const GemvArgsB& a, const GemvPlanB& p, cudaStream_t stream) {
    switch (p.passes) {
        case -4: return launch_kernel_pdl(gemv1_bl_norm_kernel<C>, a, p, stream);
        case -3: return launch_kernel_pdl(gemv1_bl_routed_kernel<C>, a, p, stream);
        case -2: return launch_kernel_pdl(gemv1_bl_swiglu_kernel<C>, a, p, stream);
        case -1: return p.multi ? launch_kernel_pdl(gemv1_bl_multi_kernel<C>, a, p, stream, *p.multi) : cudaErrorInvalidValue;
        case 0:
            if (a.glu || a.reduce.world > 0 || !C::PLAIN_FORM) return launch_kernel_pdl(gemv1_bl_epi_kernel<C>, a, p, stream);
            if (a.route_ids == nullptr && p.grid_y == 1 && p.grid == a.w.nrb && a.private_sums) return launch_kernel_pdl(gemv1_bl_one_kernel<C>, a, p, stream);
            return launch_kernel_pdl(gemv1_bl_kernel<C>, a, p, stream);
        case 1: return launch_kernel_pdl(gemvn_bl_kernel<C, 1>, a, p, stream);
        case 2: return launch_kernel_pdl(gemvn_bl_kernel<C, 2>, a, p, stream);
        case 4: return launch_kernel_pdl(gemvn_bl_kernel<C, 4>, a, p, stream);
        case 108: return launch_kernel_pdl(gemvh_bl_kernel<C, 1>, a, p, stream);
        case 116: return launch_kernel_pdl(gemvh_bl_kernel<C, 2>, a, p, stream);
        default: return cudaErrorInvalidValue;
    }
}
template <int BITS, int T>
static cudaError_t launch_gemv_bl_one(const GemvArgsB& a, const GemvPlanB& p, cudaStream_t stream) {
    return launch_gemv_codec<NintCodec<BITS, T>>(a, p, stream);
}

#define MFQB_GEMV_BL_INSTANTIATE(BITS)                                                                              \
    template <int T>                                                                                                \
    static cudaError_t launch_if_catalog(const GemvArgsB& a, const GemvPlanB& p, cudaStream_t stream) {             \
        if constexpr (nint_bl_in_catalog(BITS, T)) return launch_gemv_bl_one<BITS, T>(a, p, stream);                \
        else return cudaErrorInvalidValue;                                                                          \
    }                                                                                                               \
    template <int T>                                                                                                \
    static cudaError_t launch_s_if_catalog(const GemvSArgs& a, const GemvSPlan& p, cudaStream_t stream) {           \
        if constexpr (nint_bl_in_catalog(BITS, T)) return launch_gemvs_codec<NintCodec<BITS, T>>(a, p, stream);     \
        else return cudaErrorInvalidValue;                                                                          \
    }                                                                                                               \
    template <>                                                                                                     \
    cudaError_t launch_gemvs_bits<BITS>(const GemvSArgs& a, const GemvSPlan& p, cudaStream_t stream) {              \
        switch (a.w.t8) {                                                                                           \
            case 2: return launch_s_if_catalog<2>(a, p, stream);                                                    \
            case 3: return launch_s_if_catalog<3>(a, p, stream);                                                    \
            case 4: return launch_s_if_catalog<4>(a, p, stream);                                                    \
            case 5: return launch_s_if_catalog<5>(a, p, stream);                                                    \
            case 6: return launch_s_if_catalog<6>(a, p, stream);                                                    \
            case 8: return launch_s_if_catalog<8>(a, p, stream);                                                    \
            default: return cudaErrorInvalidValue;                                                                  \
        }                                                                                                           \
    }                                                                                                               \
    template <>                                                                                                     \
    cudaError_t launch_gemv_bl_bits<BITS>(const GemvArgsB& a, const GemvPlanB& p, cudaStream_t stream) {            \
        switch (a.w.t8) {                                                                                           \
            case 2: return launch_if_catalog<2>(a, p, stream);                                                      \
            case 3: return launch_if_catalog<3>(a, p, stream);                                                      \
            case 4: return launch_if_catalog<4>(a, p, stream);                                                      \
            case 5: return launch_if_catalog<5>(a, p, stream);                                                      \
            case 6: return launch_if_catalog<6>(a, p, stream);                                                      \
            case 8: return launch_if_catalog<8>(a, p, stream);                                                      \
            default: return cudaErrorInvalidValue;                                                                  \
        }                                                                                                           \
    }

}  // namespace mfqb
