// Lane-field bit packing shared by the host-side packers and the device kernels.
//
// A 32-bit register is seen as 32/W lanes of W bits (W = 8: the four bytes of an int8
// tensor-core operand; W = 16: the two halves of a 16-bit pair operand).  A "field" is one
// unsigned code of B bits per lane, all at the same position of their lanes, so a single
// shift + mask yields a register whose every lane holds its code at bit 0.  A unit of U words
// stores NP fields with no wasted bits:
//
//   * every word holds F = W / B fields at lane bits [f*B, f*B+B);
//   * the L = W - F*B left-over bits at the top of each lane, taken word after word, form a
//     second little-endian stream per lane that holds the remaining (U*L)/B fields.
//
//   W = 8    B : 2  3  4  5  6  8            W = 16   B : 1  2  3  4  5  6  7  8
//            U : 1  3  1  5  3  1                     U : 1  1  3  1  5  3  7  1
//            NP: 4  8  2  8  4  1                     NP: 16 8 16  4 16  8 16  2
//
// The same code runs on the host (pack, and unpack for self-checks) and in kernels (unpack
// with compile-time field indices, so every shift and mask is an immediate).
#pragma once
#include <cstdint>

#if defined(__CUDACC__)
#define MFQB_HD __host__ __device__ __forceinline__
#define MFQB_HDC __host__ __device__
#else
#define MFQB_HD inline
#define MFQB_HDC
#endif

namespace mfqb {

constexpr int lane_unit_gcd(int a, int b) { return b == 0 ? a : lane_unit_gcd(b, a % b); }

template <int B, int W>
struct LaneUnit {
    static_assert(W == 8 || W == 16, "lane width");
    static_assert(B >= 1 && B <= W, "code width");
    static constexpr uint32_t REP = W == 8 ? 0x01010101u : 0x00010001u;   // bit 0 of every lane
    static constexpr int F = W / B;                 // fields per word
    static constexpr int L = W - F * B;             // left-over bits per lane per word
    static constexpr int U = L == 0 ? 1 : B / lane_unit_gcd(B, L);   // words per unit (U*L is a multiple of B)
    static constexpr int EXTRA = (U * L) / B;       // fields rebuilt from the left-over bits
    static constexpr int NP = U * F + EXTRA;        // fields per unit
    static constexpr uint32_t MASK = ((1u << B) - 1u) * REP;

    // Field t of a sequence of whole units starting at w.  Meant for fully unrolled kernel
    // loops: once t is a compile-time constant every index, shift and mask folds.
    static MFQB_HD uint32_t at(const uint32_t* w, int t) {
        const uint32_t* u = w + (t / NP) * U;
        const int tt = t % NP;
        if (tt < U * F) return (u[tt / F] >> ((tt % F) * B)) & MASK;
        // bits [e*B, e*B+B) of the left-over stream; word i contributes stream bits
        // [i*L, i*L+L), stored at bits [F*B, W) of each lane
        const int e = tt - U * F, lo = e * B, hi = e * B + B;
        uint32_t r = 0;
#pragma unroll
        for (int i = 0; i < U; ++i) {
            const int s0 = i * L, s1 = i * L + L;
            const int a = s0 > lo ? s0 : lo, b = s1 < hi ? s1 : hi;
            if (a < b) {
                const int src = F * B + (a - s0), dst = a - lo;
                const uint32_t m = (((1u << (b - a)) - 1u) * REP) << dst;
                r |= (src >= dst) ? ((u[i] >> (src - dst)) & m) : ((u[i] << (dst - src)) & m);
            }
        }
        return r;
    }

    // Host: store field t (codes at bit 0 of each lane of v) into zero-initialised units.
    static inline void put(uint32_t* w, int t, uint32_t v) {
        uint32_t* u = w + (t / NP) * U;
        const int tt = t % NP;
        if (tt < U * F) {
            u[tt / F] |= v << ((tt % F) * B);
            return;
        }
        if constexpr (L > 0) {
            const int e = tt - U * F;
            for (int bit = 0; bit < B; ++bit) {
                const int s = e * B + bit, i = s / L, off = F * B + (s % L);
                u[i] |= ((v >> bit) & REP) << off;
            }
        }
    }

    // Words needed for n fields (whole units).
    MFQB_HDC static constexpr int words_for(int nfields) { return (nfields + NP - 1) / NP * U; }
};

template <int B>
using ByteUnit = LaneUnit<B, 8>;

// Run-time dispatch helpers for host code (byte lanes).
inline int byte_unit_words(int bits, int nfields) {
    switch (bits) {
        case 2: return ByteUnit<2>::words_for(nfields);
        case 3: return ByteUnit<3>::words_for(nfields);
        case 4: return ByteUnit<4>::words_for(nfields);
        case 5: return ByteUnit<5>::words_for(nfields);
        case 6: return ByteUnit<6>::words_for(nfields);
        default: return ByteUnit<8>::words_for(nfields);
    }
}
inline void byte_unit_put(int bits, uint32_t* w, int t, uint32_t v) {
    switch (bits) {
        case 2: ByteUnit<2>::put(w, t, v); break;
        case 3: ByteUnit<3>::put(w, t, v); break;
        case 4: ByteUnit<4>::put(w, t, v); break;
        case 5: ByteUnit<5>::put(w, t, v); break;
        case 6: ByteUnit<6>::put(w, t, v); break;
        default: ByteUnit<8>::put(w, t, v); break;
    }
}
inline uint32_t byte_unit_get(int bits, const uint32_t* w, int t) {
    switch (bits) {
        case 2: return ByteUnit<2>::at(w, t);
        case 3: return ByteUnit<3>::at(w, t);
        case 4: return ByteUnit<4>::at(w, t);
        case 5: return ByteUnit<5>::at(w, t);
        case 6: return ByteUnit<6>::at(w, t);
        default: return ByteUnit<8>::at(w, t);
    }
}

}  // namespace mfqb
