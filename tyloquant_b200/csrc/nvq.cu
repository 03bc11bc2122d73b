// NVQ3 (D4 lattice vector quantization) on the device: handle, bit-exact decoder, GEMV.
//   w[n, k] = (+-code[index][k % 4]) * (anchor[n] * s[n, k / 24])
// Replaces nvq_dequant_kernel / nvq_gemv_* (mfq/kernels/cuda/nvq_matmul.cu:421-471, 1057-1219)
// on the int8 tensor-core kernels shared with NINT (activations quantised per group to int16 planes).
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <algorithm>

#include "cuda_util.h"
#include "nvq.h"
#include "nvq_blayout.h"

namespace mfqb {

void launch_bl_gemv(const NintDevB& w, const void* x, int m, void* y, int y_dtype, int ldy, int device, cudaStream_t s, bool swiglu = false, bool glu = false);

struct NvqDevice {
    NintDevB d{};
    DevBuf items, anchors, table;
    int device = 0;
};
void NvqDeviceDeleter::operator()(NvqDevice* p) const { delete p; }
const NintDevB& nvq_device_layout(const NvqDevice& w) { return w.d; }

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
    if ((size_t)t.banks * t.entries * 64 > 128 * 1024)
        fail(MFQB_ERR_UNSUPPORTED, "NVQ codebook of %d banks x %d entries is too large for the shared-memory table", t.banks, t.entries);
    NvqPackedB p = pack_nvq_bytes(t);
    NvqDevicePtr w(new NvqDevice);
    DeviceGuard guard(device);
    w->device = device;
    w->items.upload(p.items.data(), p.items.size() * 4);
    w->anchors.upload(p.anchors.data(), p.anchors.size() * 4);
    w->table.upload(p.table.data(), p.table.size() * 4);
    w->d = p.d;
    w->d.items = static_cast<const uint32_t*>(w->items.p);
    w->d.anchors = static_cast<const uint32_t*>(w->anchors.p);
    w->d.table = static_cast<const uint32_t*>(w->table.p);
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
        info->device_bytes = w->items.bytes + w->anchors.bytes + w->table.bytes;
    }
    return w;
}

// ---- reference decoder on the GPU -----------------------------------------------------------
// One thread per (row, group, vector).  w = fl(signed_code * fl(anchor * s)): two separately
// rounded float32 products, as nvq_quant.dequantize / dequantize_nvq_jsc compute it
// (mfq/quantize/nvq_quant.py:612-626, mfq/quantize/nvq_jsc.py:1053-1079).
__global__ void nvq_bl_dequant_kernel(const NintDevB w, void* out, int out_dtype) {
    const int fb = w.index_bits + 4;
    const size_t total = (size_t)w.n * w.ng * 6;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
        const int v = (int)(idx % 6);
        const size_t rg = idx / 6;
        const int grp = (int)(rg % w.ng), row = (int)(rg / w.ng);
        const int rb = row >> 4, q = row & 7, hi = (row >> 3) & 1, ch = grp / kChunkGroupsB, g = grp % kChunkGroupsB;
        const int f = g >> 2, o = g & 3;
        const int lane = 4 * q + 2 * (o & 1) + (v & 1);
        const int reg = (f * 3 + (v >> 1)) * 4 + 2 * (o >> 1) + hi;
        const uint32_t* rec = w.items + ((size_t)rb * w.nchunks + ch) * w.rec_words;
        const int pos = reg * fb, wi = pos >> 5, sh = pos & 31;
        unsigned long long bits = rec[wi * 32 + lane];
        if (sh + fb > 32) bits |= (unsigned long long)rec[(wi + 1) * 32 + lane] << 32;
        const uint32_t field = (uint32_t)(bits >> sh) & ((1u << fb) - 1u);
        const uint32_t state = (rec[w.wc * 32 + 4 * q + (g >> 1)] >> (8 * (2 * hi + (g & 1)))) & 15u;
        const float anchor = __half2float(__ushort_as_half((unsigned short)(w.anchors[row] & 0xFFFFu)));
        const float scale = __fmul_rn(anchor, w.jsc ? w.lut[state] : (float)state);
        const uint32_t bank = (w.bankmap >> (2 * state)) & 3u;
        const uint32_t codes = w.table[((size_t)bank * w.entries + (field >> 4)) * 16 + (field & 15u)];
        for (int j = 0; j < 4; ++j) {
            const int k = grp * 24 + v * 4 + j;
            if (k >= w.k) break;
            const float val = __fmul_rn((float)(int)(signed char)(codes >> (8 * j)), scale);
            const size_t off = (size_t)row * w.k + k;
            if (out_dtype == MFQB_F32) reinterpret_cast<float*>(out)[off] = val;
            else reinterpret_cast<__nv_bfloat16*>(out)[off] = __float2bfloat16_rn(val);
        }
    }
}

void nvq_dequant(const NvqDevice& w, void* out, int out_dtype, cudaStream_t stream) {
    const size_t total = (size_t)w.d.n * w.d.ng * 6;
    const int block = 256, grid = (int)std::min<size_t>((total + block - 1) / block, 148 * 16);
    nvq_bl_dequant_kernel<<<grid, block, 0, stream>>>(w.d, out, out_dtype);
    MFQB_CUDA(cudaGetLastError());
}

void nvq_mul_mat(const NvqDevice& w, const void* x_bf16, int m, void* y, int y_dtype, cudaStream_t stream) {
    const size_t ysz = y_dtype == MFQB_F32 ? 4 : 2;
    for (int m0 = 0; m0 < m; m0 += 8) {   // batch rows one launch covers
        const int mm = std::min(8, m - m0);
        launch_bl_gemv(w.d, static_cast<const char*>(x_bf16) + (size_t)m0 * w.d.k * 2, mm, static_cast<char*>(y) + (size_t)m0 * w.d.n * ysz,
                       y_dtype, w.d.n, w.device, stream);
    }
}

}  // namespace mfqb
