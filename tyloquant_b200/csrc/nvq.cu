// NVQ3 (D4 lattice vector quantization) on the device: handle, bit-exact decoder, GEMV.
//   w[n, k] = (+-code[index][k % 4]) * (anchor[n] * s[n, k / 24])
// Replaces nvq_dequant_kernel / nvq_gemv_* (mfq/kernels/cuda/nvq_matmul.cu:421-471, 1057-1219)
// without their int8 activation quantization.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <algorithm>

#include "cuda_util.h"
#include "nint_gemv_m1.cuh"
#include "nvq.h"
#include "nvq_layout.h"

namespace mfqb {

uint64_t selfcheck_nvq_layout(const HostNvq& t);

struct NvqDevice {
    NvqDev d{};
    DevBuf items, anchors, cb;
    int device = 0;
};
void NvqDeviceDeleter::operator()(NvqDevice* p) const { delete p; }

void check_nvq_dtype(const std::string& dtype, const HostNvq& t) {
    const std::string d = dtype == "NIQ3" ? "NVQ3" : dtype;
    const bool want_jsc = d != "NVQ3";
    if (want_jsc != t.jsc)
        fail(MFQB_ERR_FORMAT, "MFQ dtype/blob mismatch: %s %s the JSC profile", dtype.c_str(), want_jsc ? "lacks" : "contains");
    const int want_bits = d == "NVQ3J-512" ? 9 : (d == "NVQ3J-L" ? 10 : 8);
    if (want_bits != t.index_bits)
        fail(MFQB_ERR_FORMAT, "MFQ dtype/blob mismatch: %s contains a %d-entry codebook", dtype.c_str(), t.entries);
}

NvqDevicePtr make_nvq_device(const HostNvq& t, int device, mfqb_weight_info* info) {
    NvqPacked p = pack_nvq_device(t);
    NvqDevicePtr w(new NvqDevice);
    DeviceGuard guard(device);
    w->device = device;
    w->items.upload(p.items.data(), p.items.size() * 4);
    w->anchors.upload(p.anchors.data(), p.anchors.size() * 4);
    w->cb.upload(p.cb.data(), p.cb.size() * 4);
    w->d = p.d;
    w->d.items = static_cast<const uint32_t*>(w->items.p);
    w->d.anchors = static_cast<const uint32_t*>(w->anchors.p);
    w->d.cb = static_cast<const NvqPair*>(w->cb.p);
    if (info) {
        info->family = MFQB_FAMILY_NVQ;
        info->bits = t.index_bits;
        info->groupsize = t.gs;
        info->sub_bits = t.sub_bits;
        info->n = t.n;
        info->k = t.k;
        info->device = device;
        info->jsc_banks = t.jsc ? t.banks : 0;
        info->payload_bytes = nvq_payload_bytes(t);
        info->device_bytes = w->items.bytes + w->anchors.bytes + w->cb.bytes;
    }
    return w;
}

// ---- reference decoder on the GPU -----------------------------------------------------------
// One thread per (row, group).  w = fl(signed_code * fl(anchor * s)): two separately rounded
// float32 products, as nvq_quant.dequantize / dequantize_nvq_jsc compute it
// (mfq/quantize/nvq_quant.py:612-626, mfq/quantize/nvq_jsc.py:1053-1079).
__global__ void nvq_dequant_kernel(const NvqDev w, void* out, int out_dtype) {
    const size_t total = (size_t)w.n * w.ng;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
        const int grp = (int)(idx % w.ng), row = (int)(idx / w.ng);
        const int rb = row >> 4, q = row & 7, r = (row >> 3) & 1, ch = grp / kNvqChunkGroups, g = grp % kNvqChunkGroups;
        const uint32_t* rec = w.items + ((size_t)rb * w.nchunks + ch) * w.rec_words;
        const uint32_t sword = rec[w.wc * 32 + (g >> 2) * 8 + q];
        const uint32_t state = (sword >> ((g & 3) * 4 + 16 * r)) & 15u;
        const float anchor = __half2float(__ushort_as_half((unsigned short)(w.anchors[row] & 0xFFFFu)));
        const float s = w.jsc ? w.lut[state] : (float)state;
        const float scale = __fmul_rn(anchor, s);
        const uint32_t bank = (w.bankmap >> (2 * state)) & 3u;
        const int pr = g >> 1, h = g & 1;
        for (int v = 0; v < 6; ++v) {
            int c, u;
            if (h == 0) { if (v < 4) { c = v; u = 0; } else { c = v - 4; u = 1; } }
            else { if (v < 2) { c = v + 2; u = 1; } else { c = v - 2; u = 2; } }
            const int pos = ((pr * 2 + r) * 3 + u) * w.fb, wi = pos >> 5, sh = pos & 31, lane = 4 * q + c;
            unsigned long long bits = rec[wi * 32 + lane];
            if (sh + w.fb > 32) bits |= (unsigned long long)rec[(wi + 1) * 32 + lane] << 32;
            const uint32_t f = (uint32_t)(bits >> sh) & ((1u << w.fb) - 1u);
            const uint32_t index = f & ((1u << w.index_bits) - 1u), sg = f >> w.index_bits;
            const NvqPair e = w.cb[bank * w.entries + index];
            const uint32_t pair[2] = {e.x, e.y};
            for (int j = 0; j < 4; ++j) {
                const int k = grp * kNvqGroup + v * 4 + j;
                if (k >= w.k) break;
                float code = __uint_as_float(((pair[j >> 1] >> ((j & 1) * 16)) & 0xFFFFu) << 16);
                if ((sg >> j) & 1u) code = -code;
                const float val = __fmul_rn(code, scale);
                const size_t o = (size_t)row * w.k + k;
                if (out_dtype == MFQB_F32) reinterpret_cast<float*>(out)[o] = val;
                else reinterpret_cast<__nv_bfloat16*>(out)[o] = __float2bfloat16_rn(val);
            }
        }
    }
}

void nvq_dequant(const NvqDevice& w, void* out, int out_dtype, cudaStream_t stream) {
    const size_t total = (size_t)w.d.n * w.d.ng;
    const int block = 256, grid = (int)std::min<size_t>((total + block - 1) / block, 148 * 16);
    nvq_dequant_kernel<<<grid, block, 0, stream>>>(w.d, out, out_dtype);
    MFQB_CUDA(cudaGetLastError());
}

// GEMV: defined in nvq_gemv.cu
void nvq_gemv_m1(const NvqDev& w, const void* x, void* y, int y_dtype, int device, cudaStream_t stream);

void nvq_mul_mat(const NvqDevice& w, const void* x_bf16, int m, void* y, int y_dtype, cudaStream_t stream) {
    // The weight-streaming kernel takes one activation row; further rows re-stream the weight.
    const size_t ysz = y_dtype == MFQB_F32 ? 4 : 2;
    for (int i = 0; i < m; ++i)
        nvq_gemv_m1(w.d, static_cast<const char*>(x_bf16) + (size_t)i * w.d.k * 2,
                    static_cast<char*>(y) + (size_t)i * w.d.n * ysz, y_dtype, w.device, stream);
}

}  // namespace mfqb
