// Prefill GEMM for NINT weights on tcgen05 tensor cores with the accumulator in tensor memory.
//
//   y[m, n] = sum_k x[m, k] * W[n, k]           (m = tokens, large;  W packed NINT)
//
// One CTA owns a tile of 128 weight rows x BN tokens and walks K one chunk (8 groups) at a time
// through a two-stage shared-memory ring:
//   * warps 0-7 (producers): warp r dequantises the chunk's record of row-block r of the tile
//     (w = d*q - m in float32, rounded once to f16) into the A tile, and all eight warps copy the
//     BN x chunk slice of x (f16) into the B tile with 16-byte cp.async; both tiles are K-major rows
//     of 128 bytes with the 128-byte swizzle the tensor core expects;
//   * warp 8: one thread issues tcgen05.mma (M = 128, N = BN, K = 16 per instruction) for the
//     chunk, D accumulating in tensor memory, and tcgen05.commit hands the stage back;
//   * epilogue: warps 0-7 read the accumulator with tcgen05.ld (lane = weight row) and store y.
// f16 (not bf16) operands keep the dequantised weights within 2^-11 relative; x arrives as f16 from
// a conversion pre-pass.  Every mbarrier wait is bounded: on expiry the kernel records an error
// word and every role leaves through the common exit, which frees the tensor memory.
// Replaces mmq_f16_packed_kernel and the dequantise-then-cuBLAS path
// (mfq/kernels/cuda/nint_matmul.cu:8138-8372, 303-333).
#pragma once
#include <cuda.h>
#include <cuda_fp16.h>

#include <algorithm>
#include <type_traits>

#include "nint_gemv_m1.cuh"
#include "tc05.cuh"

namespace mfqb {

struct GemmArgs {
    NintDev w;
    const __half* x16;   // [m, kx] f16, kx = k rounded up to 8, zero padded
    int m, kx;
    void* y;             // [m, n]
    int y_dtype;
    int bn;              // tokens per tile: 64, 128 or 256
    int stages;          // ring depth in 64-column atoms
    int* error;          // device word: set to MFQB_ERR_TIMEOUT when a wait expires
};

constexpr int kGemmProducerWarps = 16;
constexpr int kGemmThreads = (kGemmProducerWarps + 2) * 32;   // + mma warp + x loader warp

// The ring is counted in atoms: one stage = 64 columns of K = a 128 x 64 f16 slab of W (16 KB) and
// a BN x 64 f16 slab of x, each a K-major tile with the 128-byte swizzle.  A chunk of 8 groups is
// ATOMS consecutive stages.  Two producer warps share one row-block record (groups 0-3 / 4-7).
template <int BITS, int PER, int SW>
__global__ void __launch_bounds__(kGemmThreads, 1) nint_gemm_tc_kernel(const GemmArgs a, const __grid_constant__ CUtensorMap x_map) {
    constexpr int G = kChunkGroups, HALF = PER / 2, GS = 4 * PER, KST = G * GS, ATOMS = KST / 64;
    static_assert(KST % 64 == 0, "a chunk must be whole 64-element swizzle atoms");
    using QU = PairUnit<BITS>;
    using SU = PairUnit<SW>;
    constexpr int WC = QU::words_for(G * PER), SWC = SU::words_for(16), REC = WC * 32 + SWC * 8;
    constexpr int NPROD = kGemmProducerWarps * 32;
    const NintDev& w = a.w;
    const int BN = a.bn, NS = a.stages;

    extern __shared__ unsigned char smem_raw[];
    unsigned char* tiles = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    const int stage_bytes = 128 * 128 + BN * 128;   // A atom then B atom
    __shared__ __align__(8) uint64_t full_bar[8], empty_bar[8], done_bar;
    __shared__ uint32_t tmem_base_slot;
    __shared__ int failed;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int q = lane >> 2, c = lane & 3;
    const int row0 = blockIdx.x * 128, tok0 = blockIdx.y * BN;

    if (tid == 0) {
        for (int i = 0; i < 8; ++i) {
            mbar_init(&full_bar[i], NPROD + 1);   // producers + the x loader's expect_tx arrival
            mbar_init(&empty_bar[i], 1);
        }
        mbar_init(&done_bar, 1);
        failed = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == kGemmProducerWarps) tmem_alloc(&tmem_base_slot, (uint32_t)BN);
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_d = tmem_base_slot;

    if (warp < kGemmProducerWarps) {
        // ------------------------------ producers ------------------------------
        const int rbl = warp >> 1, half = warp & 1;      // row-block of the tile, group half of the chunk
        const int rb = blockIdx.x * 8 + rbl;
        const bool rb_valid = rb < w.nrb;
        bool alive = true;
        uint32_t nq[WC], ns_[SWC];
        if (rb_valid) {
            const uint32_t* rec = w.items + (size_t)rb * w.nchunks * REC;
#pragma unroll
            for (int j = 0; j < WC; ++j) nq[j] = __ldg(rec + j * 32 + lane);
#pragma unroll
            for (int j = 0; j < SWC; ++j) ns_[j] = __ldg(rec + WC * 32 + j * 8 + q);
        }
        for (int ch = 0; ch < w.nchunks && alive; ++ch) {
            // acquire the chunk's stages
#pragma unroll
            for (int j = 0; j < ATOMS; ++j) {
                const int ai = ch * ATOMS + j, st = ai % NS, use = ai / NS;
                if (use > 0 && !mbar_wait(&empty_bar[st], (use - 1) & 1)) { failed = 1; alive = false; }
            }
            if (!alive) break;
            // weight record -> f16 rows of the A atoms (this warp: 16 rows x 4 groups)
            if (rb_valid) {
                uint32_t qw[WC], sw[SWC];
#pragma unroll
                for (int j = 0; j < WC; ++j) qw[j] = nq[j];
#pragma unroll
                for (int j = 0; j < SWC; ++j) sw[j] = ns_[j];
                if (ch + 1 < w.nchunks) {   // next record's words are requested before this one is decoded
                    const uint32_t* rec = w.items + ((size_t)rb * w.nchunks + ch + 1) * REC;
#pragma unroll
                    for (int j = 0; j < WC; ++j) nq[j] = __ldg(rec + j * 32 + lane);
#pragma unroll
                    for (int j = 0; j < SWC; ++j) ns_[j] = __ldg(rec + WC * 32 + j * 8 + q);
                }
                const uint32_t an_lo = __ldg(w.anchors + rb * 16 + q), an_hi = __ldg(w.anchors + rb * 16 + 8 + q);
                const float2 f_lo = __half22float2(*reinterpret_cast<const __half2*>(&an_lo));   // (ns, nm)
                const float2 f_hi = __half22float2(*reinterpret_cast<const __half2*>(&an_hi));
                auto do_half = [&](auto half_tag) {
                    constexpr int H = decltype(half_tag)::value;
#pragma unroll
                    for (int gg = 0; gg < 4; ++gg) {
                        constexpr int dummy = 0;
                        (void)dummy;
                        const int g = H * 4 + gg;
                        float s_lo, s_hi, m_lo[2], m_hi[2];
                        pair_to_floats<SW>(SU::at(sw, g), s_lo, s_hi);
                        pair_to_floats<SW>(SU::at(sw, 8 + g / 2), m_lo[0], m_lo[1]);       // sub-mins of row lo, groups 2*(g/2), +1
                        pair_to_floats<SW>(SU::at(sw, 12 + g / 2), m_hi[0], m_hi[1]);      // row hi
                        const float d[2] = {f_lo.x * s_lo, f_hi.x * s_hi};
                        // codes enter as 128 + q (bf16 trick), so the constant term absorbs 128 * d
                        const float off = (BITS <= 6) ? 128.f : 0.f;
                        const float mn[2] = {fmaf(off, d[0], f_lo.y * m_lo[g & 1]), fmaf(off, d[1], f_hi.y * m_hi[g & 1])};
#pragma unroll
                        for (int r = 0; r < 2; ++r) {
                            const int row = rbl * 16 + q + 8 * r;
#pragma unroll
                            for (int j = 0; j < HALF; ++j) {
                                const uint32_t raw = QU::at(qw, (g * 2 + r) * HALF + j);
                                float c0, c1;
                                if constexpr (BITS <= 6) {
                                    const uint32_t v = raw | kBf16x2_128;
                                    c0 = __uint_as_float(v << 16);
                                    c1 = __uint_as_float(v & 0xFFFF0000u);
                                } else {
                                    c0 = (float)(raw & 0xFFFFu);
                                    c1 = (float)(raw >> 16);
                                }
                                const __half2 h = __floats2half2_rn(fmaf(d[r], c0, -mn[r]), fmaf(d[r], c1, -mn[r]));
                                const int k = g * GS + c * PER + 2 * j, atom = k >> 6, kk = k & 63;
                                unsigned char* at = tiles + ((ch * ATOMS + atom) % NS) * stage_bytes;
                                *reinterpret_cast<__half2*>(at + row * 128 + (((kk >> 3) ^ q) << 4) + (kk & 7) * 2) = h;
                            }
                        }
                    }
                };
                if (half == 0) do_half(std::integral_constant<int, 0>{});
                else do_half(std::integral_constant<int, 1>{});
            } else if (half == 0) {
                // rows past the end of w: zero the row-block's 16 rows in every atom of the chunk
                for (int i = lane; i < 16 * ATOMS * 8; i += 32) {
                    const int r = i / (ATOMS * 8), rest = i % (ATOMS * 8), atom = rest >> 3, c16 = rest & 7;
                    unsigned char* at = tiles + ((ch * ATOMS + atom) % NS) * stage_bytes;
                    *reinterpret_cast<uint4*>(at + (rbl * 16 + r) * 128 + (c16 << 4)) = make_uint4(0u, 0u, 0u, 0u);
                }
            }
            fence_proxy_async_smem();
#pragma unroll
            for (int j = 0; j < ATOMS; ++j) mbar_arrive(&full_bar[(ch * ATOMS + j) % NS]);
        }
    } else if (warp == kGemmProducerWarps + 1) {
        // ------------------------------ x loader (TMA) ------------------------------
        if (lane == 0) {
            const int natoms = w.nchunks * ATOMS;
            for (int ai = 0; ai < natoms; ++ai) {
                const int st = ai % NS, use = ai / NS;
                if (use > 0 && !mbar_wait(&empty_bar[st], (use - 1) & 1)) { failed = 1; break; }
                mbar_arrive_expect_tx(&full_bar[st], (uint32_t)(BN * 128));
                tma_load_2d(tiles + st * stage_bytes + 128 * 128, &x_map, ai * 64, tok0, &full_bar[st]);
            }
        }
    } else if (lane == 0) {
        // ------------------------------ mma issuer ------------------------------
        const uint32_t idesc = instr_desc_f16(128, BN);
        const int natoms = w.nchunks * ATOMS;
        for (int ai = 0; ai < natoms; ++ai) {
            const int st = ai % NS, use = ai / NS;
            if (!mbar_wait(&full_bar[st], use & 1)) { failed = 1; break; }
            tc_fence_after_sync();
            const uint32_t a_base = smem_u32(tiles + st * stage_bytes), b_base = a_base + 128 * 128;
#pragma unroll
            for (int j = 0; j < 4; ++j)
                tc_mma_f16(tmem_d, smem_desc_sw128(a_base + j * 32), smem_desc_sw128(b_base + j * 32), idesc, ai > 0 || j > 0);
            tc_commit(&empty_bar[st]);
        }
        tc_commit(&done_bar);
    }

    // ------------------------------ epilogue ------------------------------
    if (warp < kGemmProducerWarps) {
        bool ok = !failed && mbar_wait(&done_bar, 0);
        ok = __all_sync(0xffffffffu, ok);   // tcgen05.ld is warp-wide: take the decision together
        if (!ok) failed = 1;
        tc_fence_after_sync();
        const int lane_quarter = warp & 3, part = warp >> 2;          // 4 column parts
        const int cols_per_part = BN / 4 < 32 ? 32 : BN / 4;
        const int c_begin = part * cols_per_part, c_end = min(BN, c_begin + cols_per_part);
        if (ok && c_begin < BN) {
            const int n = row0 + lane_quarter * 32 + lane;
            for (int cb = c_begin; cb < c_end; cb += 32) {
                uint32_t r[32];
                tmem_ld32(tmem_d + ((uint32_t)(lane_quarter * 32) << 16) + (uint32_t)cb, r);
                if (n < w.n) {
#pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        const int tok = tok0 + cb + i;
                        if (tok < a.m) {
                            const float v = __uint_as_float(r[i]);
                            if (a.y_dtype == 0 /* MFQB_F32 */) reinterpret_cast<float*>(a.y)[(size_t)tok * w.n + n] = v;
                            else reinterpret_cast<__nv_bfloat16*>(a.y)[(size_t)tok * w.n + n] = __float2bfloat16_rn(v);
                        }
                    }
                }
            }
        }
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == kGemmProducerWarps) {
        tmem_free(tmem_d, (uint32_t)BN);
        if (lane == 0 && failed) atomicExch(a.error, MFQB_ERR_TIMEOUT);
    }
}

struct GemmPlan {
    int bn, stages, grid_x, grid_y;
    size_t smem;
};
// gs must be 16, 24 or 32 (a chunk is then whole swizzle atoms); returns bn = 0 otherwise.
inline GemmPlan plan_nint_gemm(const NintDev& w, int m) {
    GemmPlan p{};
    if (!(w.gs == 16 || w.gs == 24 || w.gs == 32) || w.per * 4 != w.gs) return p;
    const int atoms = kChunkGroups * w.gs / 64;
    // wide token tiles amortise the dequantisation; 32-wide groups (4 atoms per chunk) take the
    // narrower tile so that the ring holds more than one chunk
    int bn = (w.gs == 32) ? 128 : 256;
    while (bn > 64 && bn / 2 >= m) bn /= 2;
    p.bn = bn;
    const int stage_bytes = 128 * 128 + bn * 128;
    p.stages = std::min(8, (int)((220 * 1024) / stage_bytes));
    if (p.stages < atoms) { p.bn = 0; return p; }
    p.grid_x = (w.n + 127) / 128;
    p.grid_y = (m + bn - 1) / bn;
    p.smem = (size_t)p.stages * stage_bytes + 1024;
    return p;
}

template <int BITS>
cudaError_t launch_nint_gemm_bits(const GemmArgs& a, const GemmPlan& p, const CUtensorMap& x_map, cudaStream_t stream);

}  // namespace mfqb
