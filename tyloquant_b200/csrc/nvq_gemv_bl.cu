// NVQ3 instantiations of the byte-lane GEMV kernels.
#include "nint_gemv_bl_launch.cuh"
#include "nvq_codec.cuh"

namespace mfqb {

cudaError_t launch_gemv_bl_nvq(const GemvArgsB& a, const GemvPlanB& p, cudaStream_t stream) {
    const NintDevB& w = a.w;
    if (w.jsc) {
        if (w.index_bits == 8) return launch_gemv_codec<NvqCodec<8, true>>(a, p, stream);
        if (w.index_bits == 9) return launch_gemv_codec<NvqCodec<9, true>>(a, p, stream);
        if (w.index_bits == 10) return launch_gemv_codec<NvqCodec<10, true>>(a, p, stream);
    } else if (w.index_bits == 8) {
        return launch_gemv_codec<NvqCodec<8, false>>(a, p, stream);
    }
    return cudaErrorInvalidValue;
}

}  // namespace mfqb
