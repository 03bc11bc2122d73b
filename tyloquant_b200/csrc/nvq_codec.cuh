// Codec of byte-lane NVQ3 records for the int8 tensor-core GEMV kernels (see nvq_blayout.h).
#pragma once
#include "nint_gemvn_bl.cuh"

namespace mfqb {

template <int IB, bool JSC>
struct NvqCodec {
    static constexpr int T = 3, FB = IB + 4, WC = (24 * FB + 31) / 32, SW = 1;
    static constexpr bool A_SIGNED = true, HAS_MIN = false, NEEDS_OWN_SCALE = JSC;
    static constexpr int QMID = 0;   // lattice codes are signed around zero
    // The stripped single-row kernel is slower than the general one for the plain (non-JSC) lattice codec:
    // 23.1 against 17.6 us on 17408 x 5120 (same registers, no spills; the table look-ups get scheduled worse).
    static constexpr bool PLAIN_FORM = JSC;
    static constexpr int MIN_CTAS = IB == 8 ? 3 : 2;
    static constexpr uint32_t OFFMASK = ((1u << FB) - 1u) << 2;   // a field as a byte offset into the signed table

    // The signed table [bank][index][nibble] (four int8 per entry) and the 16 state scales, copied
    // into shared memory once per CTA.
    struct Ctx {
        const unsigned char* table;
        const float* lut;
        uint32_t bank_bytes;
        __device__ __forceinline__ void init(unsigned char* smem, const NintDevB& w, int tid, int nthreads) {
            uint4* dst = reinterpret_cast<uint4*>(smem);
            const uint4* src = reinterpret_cast<const uint4*>(w.table);
            for (int i = tid; i < w.table_words / 4; i += nthreads) dst[i] = __ldg(src + i);
            float* l = reinterpret_cast<float*>(smem + (size_t)w.table_words * 4);
            if (tid < 16) l[tid] = w.lut[tid];
            table = smem;
            lut = l;
            bank_bytes = (uint32_t)w.entries * 64u;
        }
    };
    __host__ __device__ static size_t ctx_bytes(const NintDevB& w) { return (size_t)w.table_words * 4 + 64; }

    __device__ static __forceinline__ uint32_t areg(const uint32_t* qw, int r, const Ctx& ctx, const uint32_t* own) {
        const int pos = r * FB, wi = pos >> 5, sh = pos & 31;
        uint32_t off;
        if (sh + FB <= 32) off = sh >= 2 ? (qw[wi] >> (sh - 2)) & OFFMASK : (qw[wi] << (2 - sh)) & OFFMASK;
        else off = __funnelshift_r(qw[wi], qw[wi + 1], sh - 2) & OFFMASK;   // a field that straddles two words starts above bit 2
        if constexpr (JSC) {
            const int i = (r / 12) * 4 + (r & 3);   // (family, register of the step): the (row, group) pair of this register
            off += ((own[0] >> (8 * (i >> 1) + 4 + 2 * (i & 1))) & 3u) * ctx.bank_bytes;
        }
        return *reinterpret_cast<const uint32_t*>(ctx.table + off);
    }
    __device__ static __forceinline__ void scales(const uint32_t* sw, const Ctx& ctx, float (&ss)[4], float (&sm)[4]) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const uint32_t st = (sw[0] >> (8 * i)) & 15u;
            ss[i] = JSC ? ctx.lut[st] : (float)st;
            sm[i] = 0.f;
        }
    }
};

}  // namespace mfqb
