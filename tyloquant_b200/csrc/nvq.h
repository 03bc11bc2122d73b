// NVQ3 (D4 lattice vector quantization) device weights: interface used by weights.cu.
#pragma once
#include <memory>
#include <string>

#include "common.h"

typedef struct CUstream_st* cudaStream_t;

namespace mfqb {

struct NvqDevice;
struct NvqDeviceDeleter { void operator()(NvqDevice* p) const; };
using NvqDevicePtr = std::unique_ptr<NvqDevice, NvqDeviceDeleter>;

void check_nvq_dtype(const std::string& dtype, const HostNvq& t);
NvqDevicePtr make_nvq_device(const HostNvq& t, int device, mfqb_weight_info* info);
struct NintDevB;
const NintDevB& nvq_device_layout(const NvqDevice& w);
void nvq_dequant(const NvqDevice& w, void* out, int out_dtype, cudaStream_t stream);
void nvq_mul_mat(const NvqDevice& w, const void* x_bf16, int m, void* y, int y_dtype, cudaStream_t stream);

}  // namespace mfqb
