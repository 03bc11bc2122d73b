// NINT8 instantiations of the tcgen05 prefill GEMM.
#include "nint_gemm_tc.cuh"

namespace mfqb {
MFQB_GEMM_INSTANTIATE(8)
}  // namespace mfqb
