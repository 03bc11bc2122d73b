// NINT4 instantiations of the byte-lane GEMV kernels.
#include "nint_gemv_bl_launch.cuh"

namespace mfqb {
MFQB_GEMV_BL_INSTANTIATE(4)
}  // namespace mfqb
