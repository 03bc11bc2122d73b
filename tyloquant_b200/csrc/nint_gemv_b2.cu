// NINT2 instantiations of the weight-streaming GEMV (one translation unit per code width
// so the widths compile in parallel).
#include "nint_gemv.cuh"

namespace mfqb {

template <int BITS, int PER, int SW>
static cudaError_t launch_one(const GemvArgs& a, const GemvPlan& p, cudaStream_t stream) {
    auto kern = nint_gemv_kernel<BITS, PER, SW>;
    if (p.smem > 48 * 1024) {
        const cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)p.smem);
        if (e != cudaSuccess) return e;
    }
    kern<<<p.grid, kGemvThreads, p.smem, stream>>>(a);
    return cudaGetLastError();
}

template <>
cudaError_t launch_nint_gemv_bits<2>(const GemvArgs& a, const GemvPlan& p, cudaStream_t stream) {
    switch (a.w.per * 16 + a.w.sw) {
        case 69: return launch_one<2, 4, 5>(a, p, stream);
        case 72: return launch_one<2, 4, 8>(a, p, stream);
        default: return cudaErrorInvalidValue;
    }
}

}  // namespace mfqb
