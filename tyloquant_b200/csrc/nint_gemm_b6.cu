// NINT6 instantiations of the tcgen05 prefill GEMM.
#include "nint_gemm_tc.cuh"

namespace mfqb {

template <int BITS, int PER, int SW>
static cudaError_t launch_one(const GemmArgs& a, const GemmPlan& p, const CUtensorMap& x_map, cudaStream_t stream) {
    auto kern = nint_gemm_tc_kernel<BITS, PER, SW>;
    const cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)p.smem);
    if (e != cudaSuccess) return e;
    kern<<<dim3((unsigned)p.grid_x, (unsigned)p.grid_y), kGemmThreads, p.smem, stream>>>(a, x_map);
    return cudaGetLastError();
}

template <>
cudaError_t launch_nint_gemm_bits<6>(const GemmArgs& a, const GemmPlan& p, const CUtensorMap& x_map, cudaStream_t stream) {
    if (a.w.sw != 7) return cudaErrorNotSupported;
    switch (a.w.per) {
        case 6: return launch_one<6, 6, 7>(a, p, x_map, stream);
        case 8: return launch_one<6, 8, 7>(a, p, x_map, stream);
        default: return cudaErrorNotSupported;
    }
}

}  // namespace mfqb
