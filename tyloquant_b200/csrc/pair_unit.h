// Pair-field bit packing shared by the host-side packers and the device kernels.
//
// A "pair" is two unsigned codes of B bits that a kernel wants side by side in the two
// 16-bit halves of one 32-bit register (the shape of a bf16x2 tensor-core operand).  A
// unit of U 32-bit words stores NP pairs with no wasted bits:
//
//   * every word holds F = 16 / B "field pairs": pair f of the word has its low code at
//     bits [f*B, f*B+B) and its high code at the same position of the upper half, so a
//     single shift + mask yields both codes already in place;
//   * the L = 16 - F*B left-over bits at the top of each half, taken word after word, form
//     a second little-endian stream per half that holds the remaining (U*L)/B pairs.
//
//   B : 1  2  3  4  5  6  7  8
//   U : 1  1  3  1  5  3  7  1
//   NP: 16 8 16  4 16  8 16  2
//
// The same code runs on the host (pack, and unpack for self-checks) and in kernels
// (unpack with compile-time pair indices, so every shift and mask is an immediate).
#pragma once
#include <cstdint>

#if defined(__CUDACC__)
#define MFQB_HD __host__ __device__ __forceinline__
#else
#define MFQB_HD inline
#endif

namespace mfqb {

template <int B>
struct PairUnit {
    static_assert(B >= 1 && B <= 8, "code width");
    static constexpr int F = 16 / B;          // field pairs per word
    static constexpr int L = 16 - F * B;      // left-over bits per half per word
    static constexpr int U = (L == 0) ? 1 : B;  // words per unit (U*L is a multiple of B)
    static constexpr int EXTRA = (U * L) / B;   // pairs rebuilt from the left-over bits
    static constexpr int NP = U * F + EXTRA;    // pairs per unit
    static constexpr uint32_t MASK = ((1u << B) - 1u) * 0x00010001u;

    // Pair T of the unit, codes in bits [0,B) and [16,16+B).
    template <int T>
    static MFQB_HD uint32_t get(const uint32_t* w) {
        static_assert(T >= 0 && T < NP, "pair index");
        if constexpr (T < U * F) {
            constexpr int word = T / F, sh = (T % F) * B;
            return (w[word] >> sh) & MASK;
        } else {
            // bits [e*B, e*B+B) of the left-over stream; word u contributes stream bits
            // [u*L, u*L+L), stored at bits [F*B, 16) of each half.
            constexpr int e = T - U * F;
            uint32_t r = 0;
#pragma unroll
            for (int u = 0; u < U; ++u) {
                constexpr int lo = e * B, hi = e * B + B;
                const int s0 = u * L, s1 = u * L + L;       // stream range of this word
                const int a = s0 > lo ? s0 : lo, b = s1 < hi ? s1 : hi;
                if (a < b) {
                    const int src = F * B + (a - s0);       // bit inside the half
                    const int dst = a - lo;                 // bit inside the code
                    const uint32_t m = ((1u << (b - a)) - 1u) * 0x00010001u;
                    const uint32_t piece = (src >= dst) ? ((w[u] >> (src - dst)) & (m << dst))
                                                        : ((w[u] << (dst - src)) & (m << dst));
                    r |= piece;
                }
            }
            return r;
        }
    }

    // Pair t of a sequence of whole units starting at w.  Meant for fully unrolled kernel
    // loops: once t is a compile-time constant every index, shift and mask folds.
    static MFQB_HD uint32_t at(const uint32_t* w, int t) {
        const uint32_t* u = w + (t / NP) * U;
        const int tt = t % NP;
        if (tt < U * F) return (u[tt / F] >> ((tt % F) * B)) & MASK;
        const int e = tt - U * F, lo = e * B, hi = e * B + B;
        uint32_t r = 0;
#pragma unroll
        for (int i = 0; i < U; ++i) {
            const int s0 = i * L, s1 = i * L + L;
            const int a = s0 > lo ? s0 : lo, b = s1 < hi ? s1 : hi;
            if (a < b) {
                const int src = F * B + (a - s0), dst = a - lo;
                const uint32_t m = (((1u << (b - a)) - 1u) * 0x00010001u) << dst;
                r |= (src >= dst) ? ((u[i] >> (src - dst)) & m) : ((u[i] << (dst - src)) & m);
            }
        }
        return r;
    }

    // Run-time pair index (host packers / self-checks).
    static MFQB_HD uint32_t get_rt(const uint32_t* w, int t) {
        if (t < U * F) {
            const int word = t / F, sh = (t % F) * B;
            return (w[word] >> sh) & MASK;
        }
        uint32_t r = 0;
        if constexpr (L > 0) {
            const int e = t - U * F;
            for (int bit = 0; bit < B; ++bit) {
                const int s = e * B + bit, u = s / L, off = F * B + (s % L);
                r |= ((w[u] >> off) & 0x00010001u) << bit;
            }
        }
        return r;
    }

    // Host: store pair t = (lo, hi) into a zero-initialised unit.
    static inline void put(uint32_t* w, int t, uint32_t lo, uint32_t hi) {
        if (t < U * F) {
            const int word = t / F, sh = (t % F) * B;
            w[word] |= (lo << sh) | (hi << (sh + 16));
            return;
        }
        if constexpr (L > 0) {
            const int e = t - U * F;
            for (int bit = 0; bit < B; ++bit) {
                const int s = e * B + bit, u = s / L, off = F * B + (s % L);
                w[u] |= (((lo >> bit) & 1u) << off) | (((hi >> bit) & 1u) << (off + 16));
            }
        }
    }

    // Words needed for n pairs (whole units).
#if defined(__CUDACC__)
    __host__ __device__
#endif
    static constexpr int words_for(int npairs) { return (npairs + NP - 1) / NP * U; }
};

// Run-time dispatch helpers for host code.
inline int pair_unit_words(int bits, int npairs) {
    switch (bits) {
        case 1: return PairUnit<1>::words_for(npairs);
        case 2: return PairUnit<2>::words_for(npairs);
        case 3: return PairUnit<3>::words_for(npairs);
        case 4: return PairUnit<4>::words_for(npairs);
        case 5: return PairUnit<5>::words_for(npairs);
        case 6: return PairUnit<6>::words_for(npairs);
        case 7: return PairUnit<7>::words_for(npairs);
        default: return PairUnit<8>::words_for(npairs);
    }
}

template <int B>
inline void pair_put_seq(uint32_t* w, int t, uint32_t lo, uint32_t hi) {
    PairUnit<B>::put(w + (t / PairUnit<B>::NP) * PairUnit<B>::U, t % PairUnit<B>::NP, lo, hi);
}
inline void pair_put(int bits, uint32_t* w, int t, uint32_t lo, uint32_t hi) {
    switch (bits) {
        case 1: pair_put_seq<1>(w, t, lo, hi); break;
        case 2: pair_put_seq<2>(w, t, lo, hi); break;
        case 3: pair_put_seq<3>(w, t, lo, hi); break;
        case 4: pair_put_seq<4>(w, t, lo, hi); break;
        case 5: pair_put_seq<5>(w, t, lo, hi); break;
        case 6: pair_put_seq<6>(w, t, lo, hi); break;
        case 7: pair_put_seq<7>(w, t, lo, hi); break;
        default: pair_put_seq<8>(w, t, lo, hi); break;
    }
}
template <int B>
inline uint32_t pair_get_seq(const uint32_t* w, int t) {
    return PairUnit<B>::get_rt(w + (t / PairUnit<B>::NP) * PairUnit<B>::U, t % PairUnit<B>::NP);
}
inline uint32_t pair_get(int bits, const uint32_t* w, int t) {
    switch (bits) {
        case 1: return pair_get_seq<1>(w, t);
        case 2: return pair_get_seq<2>(w, t);
        case 3: return pair_get_seq<3>(w, t);
        case 4: return pair_get_seq<4>(w, t);
        case 5: return pair_get_seq<5>(w, t);
        case 6: return pair_get_seq<6>(w, t);
        case 7: return pair_get_seq<7>(w, t);
        default: return pair_get_seq<8>(w, t);
    }
}

}  // namespace mfqb
