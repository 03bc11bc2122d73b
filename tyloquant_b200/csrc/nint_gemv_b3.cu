// NINT3 instantiations of the weight-streaming GEMV (one translation unit per code width
// so the widths compile in parallel).
#include "nint_gemv_m1.cuh"

namespace mfqb {

template <int BITS, int PER, int SW>
static cudaError_t launch_one(const GemvArgs& a, const GemvPlan& p, cudaStream_t stream) {
    if (p.smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(nint_gemv_kernel<BITS, PER, SW>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)p.smem);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(nint_gemv_m1_kernel<BITS, PER, SW>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)p.smem);
        if (e != cudaSuccess) return e;
    }
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
    if (a.m == 1) return cudaLaunchKernelEx(&cfg, nint_gemv_m1_kernel<BITS, PER, SW>, a);
    return cudaLaunchKernelEx(&cfg, nint_gemv_kernel<BITS, PER, SW>, a);
}

template <>
cudaError_t launch_nint_gemv_bits<3>(const GemvArgs& a, const GemvPlan& p, cudaStream_t stream) {
    switch (a.w.per * 16 + a.w.sw) {
        case 101: return launch_one<3, 6, 5>(a, p, stream);
        case 104: return launch_one<3, 6, 8>(a, p, stream);
        default: return cudaErrorInvalidValue;
    }
}

}  // namespace mfqb
