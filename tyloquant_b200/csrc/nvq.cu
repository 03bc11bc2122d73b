// placeholder, replaced below
#include "cuda_util.h"
#include "nvq.h"
namespace mfqb {
struct NvqDevice {};
void NvqDeviceDeleter::operator()(NvqDevice* p) const { delete p; }
void check_nvq_dtype(const std::string&, const HostNvq&) {}
NvqDevicePtr make_nvq_device(const HostNvq&, int, mfqb_weight_info*) { fail(MFQB_ERR_UNSUPPORTED, "NVQ kernels not built yet"); }
void nvq_dequant(const NvqDevice&, void*, int, cudaStream_t) { fail(MFQB_ERR_UNSUPPORTED, "NVQ kernels not built yet"); }
void nvq_mul_mat(const NvqDevice&, const void*, int, void*, int, cudaStream_t) { fail(MFQB_ERR_UNSUPPORTED, "NVQ kernels not built yet"); }
uint64_t selfcheck_nvq_layout(const HostNvq&) { fail(MFQB_ERR_UNSUPPORTED, "NVQ kernels not built yet"); }
}
