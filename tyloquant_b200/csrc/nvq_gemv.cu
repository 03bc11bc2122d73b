// Single-row GEMV for NVQ3 weights.
//
// Same structure as the NINT single-row kernel: the eight mma columns carry the eight groups of
// a chunk (block-diagonal B), every warp streams its (row-block, chunk) records through a private
// cp.async ring, and the group scales are applied once per chunk in float32.  The A operand of a
// step is one lattice vector per lane and row: its four magnitudes come from the codebook in
// shared memory as two bf16x2 registers (exact small integers), the four sign bits are moved
// onto the bf16 sign positions with one integer multiply and one logic op per register.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <algorithm>

#include "cuda_util.h"
#include "nint_gemv_m1.cuh"
#include "nvq_layout.h"

namespace mfqb {

struct NvqGemvArgs {
    NvqDev w;
    const __nv_bfloat16* x;
    void* y;
    int y_dtype, rb_per_cta, xstride;
};

template <int NB>
__device__ __forceinline__ uint32_t bits_at(const uint32_t* w, int pos) {
    const int wi = pos >> 5, sh = pos & 31;
    const uint32_t v = (sh + NB <= 32) ? (w[wi] >> sh) : __funnelshift_r(w[wi], w[wi + 1], sh);
    return v & ((1u << NB) - 1u);
}

template <int IB, bool JSC>
__global__ void __launch_bounds__(256, 3) nvq_gemv_m1_kernel(const NvqGemvArgs a) {
    constexpr int FB = IB + 4, WC = (24 * FB + 31) / 32, REC = WC * 32 + 16;
    constexpr int S = gemv_m1_stages(REC);
    const NvqDev& w = a.w;

    extern __shared__ __align__(16) unsigned char smem[];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarps = blockDim.x >> 5;
    const int q = lane >> 2, c = lane & 3;
    float* ypart = reinterpret_cast<float*>(smem);
    uint32_t* anch = reinterpret_cast<uint32_t*>(ypart + (size_t)a.rb_per_cta * 16);
    float* lut = reinterpret_cast<float*>(anch + (size_t)a.rb_per_cta * 16);
    __nv_bfloat16* xs = reinterpret_cast<__nv_bfloat16*>(lut + 16);
    NvqPair* cb = reinterpret_cast<NvqPair*>(xs + a.xstride);
    uint32_t* ring = reinterpret_cast<uint32_t*>(cb + w.banks * w.entries) + (size_t)warp * S * REC;

    const int rb0 = (int)(((long long)blockIdx.x * w.nrb) / gridDim.x);
    const int nrb = (int)(((long long)(blockIdx.x + 1) * w.nrb) / gridDim.x) - rb0;
    const int my_segs = warp < w.nchunks ? (w.nchunks - warp + nwarps - 1) / nwarps : 0;
    const int n_mine = my_segs * nrb;
    int iss_i = 0, iss_seg = warp, iss_rbl = 0, iss_stage = 0;
    auto issue = [&]() {
        if (iss_i < n_mine) {
            const uint32_t* src = w.items + ((size_t)(rb0 + iss_rbl) * w.nchunks + iss_seg) * REC;
            uint32_t* dst = ring + iss_stage * REC;
#pragma unroll
            for (int off = 0; off < REC; off += 128)
                if (off + 128 <= REC || lane * 4 < REC - off) cp_async16(dst + off + lane * 4, src + off + lane * 4);
        }
        cp_async_commit();
        ++iss_i;
        if (++iss_rbl == nrb) { iss_rbl = 0; iss_seg += nwarps; }
        if (++iss_stage == S) iss_stage = 0;
    };

    pdl_launch_dependents();
#pragma unroll
    for (int i = 0; i < S; ++i) issue();
    for (int i = tid; i < nrb * 16; i += blockDim.x) {
        ypart[i] = 0.f;
        anch[i] = __ldg(w.anchors + rb0 * 16 + i);
    }
    if (tid < 16) lut[tid] = w.lut[tid];
    for (int i = tid; i < w.banks * w.entries; i += blockDim.x) cb[i] = w.cb[i];
    pdl_wait();
    {
        const int kp = a.xstride;
        if ((w.k & 7) == 0 && (reinterpret_cast<uintptr_t>(a.x) & 15) == 0) {
            for (int v = tid; v < kp / 8; v += blockDim.x) {
                uint4 val = make_uint4(0u, 0u, 0u, 0u);
                if (v * 8 < w.k) val = __ldg(reinterpret_cast<const uint4*>(a.x) + v);
                *reinterpret_cast<uint4*>(xs + v * 8) = val;
            }
        } else {
            for (int k = tid; k < kp; k += blockDim.x) xs[k] = k < w.k ? a.x[k] : __float2bfloat16(0.f);
        }
    }
    __syncthreads();

    const uint32_t* xw = reinterpret_cast<const uint32_t*>(xs);
    int cur_seg = -1;
    uint32_t b0[12], b1[12];   // block-diagonal B of the twelve steps of a chunk

    auto prepare_chunk = [&](int seg) {
#pragma unroll
        for (int p = 0; p < 4; ++p)
#pragma unroll
            for (int u = 0; u < 3; ++u) {
                int g, v;
                nvq_slot(p, u, c, g, v);
                const int kw = ((seg * kNvqChunkGroups + g) * kNvqGroup + v * 4) >> 1;
                const bool mine = q == g;
                b0[p * 3 + u] = mine ? xw[kw] : 0u;
                b1[p * 3 + u] = mine ? xw[kw + 1] : 0u;
            }
    };

    int seg = warp, rbl = 0, stage = 0;
    for (int i = 0; i < n_mine; ++i) {
        if (seg != cur_seg) { cur_seg = seg; prepare_chunk(seg); }
        asm volatile("cp.async.wait_group %0;\n" ::"n"(S - 1) : "memory");
        __syncwarp();
        const uint32_t* rec = ring + stage * REC;
        uint32_t qw[WC + 1], sw[2];
#pragma unroll
        for (int j = 0; j < WC; ++j) qw[j] = rec[j * 32 + lane];
        qw[WC] = 0u;
        sw[0] = rec[WC * 32 + q];
        sw[1] = rec[WC * 32 + 8 + q];
        __syncwarp();
        issue();

        float ch[4][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
        for (int p = 0; p < 4; ++p)
#pragma unroll
            for (int u = 0; u < 3; ++u) {
                uint32_t areg[2][2];
#pragma unroll
                for (int r = 0; r < 2; ++r) {
                    const uint32_t f = bits_at<FB>(qw, ((p * 2 + r) * 3 + u) * FB);
                    uint32_t index = f & ((1u << IB) - 1u);
                    const uint32_t sg = f >> IB;
                    if constexpr (JSC) {
                        // bank of the group this vector belongs to (group 2p or 2p+1 of the chunk)
                        const int gsel = u == 0 ? 2 * p : (u == 2 ? 2 * p + 1 : (c < 2 ? 2 * p : 2 * p + 1));
                        const uint32_t state = (sw[gsel >> 2] >> ((gsel & 3) * 4 + 16 * r)) & 15u;
                        index += ((w.bankmap >> (2 * state)) & 3u) << IB;
                    }
                    const NvqPair e = cb[index];
                    areg[r][0] = e.x ^ ((sg * 0x40008000u) & 0x80008000u);   // sign bits 0,1 -> bits 15,31
                    areg[r][1] = e.y ^ ((sg * 0x10002000u) & 0x80008000u);   // sign bits 2,3 -> bits 15,31
                }
                mma_k16(ch[(p * 3 + u) & 3], areg[0][0], areg[1][0], areg[0][1], areg[1][1], b0[p * 3 + u],
                        b1[p * 3 + u]);
            }
        float acc[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[e] = (ch[0][e] + ch[1][e]) + (ch[2][e] + ch[3][e]);
        // scales of rows (q, q+8) x groups (2c, 2c+1): adjacent nibbles of one scale word
        const uint32_t sv = sw[c >> 1] >> (8 * (c & 1));
        const uint32_t n_lo0 = sv & 15u, n_lo1 = (sv >> 4) & 15u, n_hi0 = (sv >> 16) & 15u, n_hi1 = (sv >> 20) & 15u;
        float s_lo0, s_lo1, s_hi0, s_hi1;
        if constexpr (JSC) {
            s_lo0 = lut[n_lo0]; s_lo1 = lut[n_lo1]; s_hi0 = lut[n_hi0]; s_hi1 = lut[n_hi1];
        } else {
            s_lo0 = (float)n_lo0; s_lo1 = (float)n_lo1; s_hi0 = (float)n_hi0; s_hi1 = (float)n_hi1;
        }
        const float a_lo = __half2float(__ushort_as_half((unsigned short)(anch[rbl * 16 + q] & 0xFFFFu)));
        const float a_hi = __half2float(__ushort_as_half((unsigned short)(anch[rbl * 16 + q + 8] & 0xFFFFu)));
        float v_lo = a_lo * fmaf(s_lo1, acc[1], s_lo0 * acc[0]);
        float v_hi = a_hi * fmaf(s_hi1, acc[3], s_hi0 * acc[2]);
        v_lo += __shfl_xor_sync(0xffffffffu, v_lo, 1);
        v_hi += __shfl_xor_sync(0xffffffffu, v_hi, 1);
        v_lo += __shfl_xor_sync(0xffffffffu, v_lo, 2);
        v_hi += __shfl_xor_sync(0xffffffffu, v_hi, 2);
        if (c == 0) {
            atomicAdd(ypart + rbl * 16 + q, v_lo);
            atomicAdd(ypart + rbl * 16 + q + 8, v_hi);
        }
        if (++rbl == nrb) { rbl = 0; seg += nwarps; }
        if (++stage == S) stage = 0;
    }
    asm volatile("cp.async.wait_group 0;\n" ::: "memory");
    __syncthreads();
    for (int i = tid; i < nrb * 16; i += blockDim.x) {
        const int row = rb0 * 16 + i;
        if (row < w.n) {
            const float v = ypart[i];
            if (a.y_dtype == 0 /* MFQB_F32 */) reinterpret_cast<float*>(a.y)[row] = v;
            else reinterpret_cast<__nv_bfloat16*>(a.y)[row] = __float2bfloat16_rn(v);
        }
    }
}

template <int IB, bool JSC>
static cudaError_t launch_nvq(const NvqGemvArgs& a, int grid, size_t smem, cudaStream_t stream) {
    if (smem > 48 * 1024) {
        const cudaError_t e = cudaFuncSetAttribute(nvq_gemv_m1_kernel<IB, JSC>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3(256);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, nvq_gemv_m1_kernel<IB, JSC>, a);
}

void nvq_gemv_m1(const NvqDev& w, const void* x, void* y, int y_dtype, int device, cudaStream_t stream) {
    NvqGemvArgs a;
    a.w = w;
    a.x = static_cast<const __nv_bfloat16*>(x);
    a.y = y;
    a.y_dtype = y_dtype;
    const int grid = std::min(w.nrb, 3 * device_sm_count(device));
    a.rb_per_cta = (w.nrb + grid - 1) / grid;
    const int kp = w.nchunks * kNvqChunkGroups * kNvqGroup;
    a.xstride = ((kp + 7) / 8) * 8;
    const size_t rec_bytes = (size_t)w.rec_words * 4;
    const size_t smem = (size_t)a.rb_per_cta * 16 * 8 + 64 + (size_t)a.xstride * 2 + (size_t)w.banks * w.entries * 8 +
                        (size_t)8 * gemv_m1_stages(w.rec_words) * rec_bytes;
    cudaError_t e = cudaErrorInvalidValue;
    if (w.jsc) {
        if (w.index_bits == 8) e = launch_nvq<8, true>(a, grid, smem, stream);
        else if (w.index_bits == 9) e = launch_nvq<9, true>(a, grid, smem, stream);
        else if (w.index_bits == 10) e = launch_nvq<10, true>(a, grid, smem, stream);
    } else if (w.index_bits == 8) {
        e = launch_nvq<8, false>(a, grid, smem, stream);
    }
    if (e != cudaSuccess) fail(MFQB_ERR_CUDA, "NVQ GEMV launch (index bits %d): %s", w.index_bits, cudaGetErrorString(e));
}

}  // namespace mfqb
