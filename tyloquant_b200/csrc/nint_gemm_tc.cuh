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
#include <cuda_fp16.h>

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
    int* error;          // device word: set to MFQB_ERR_TIMEOUT when a wait expires
};

constexpr int kGemmThreads = 288;   // 8 producer warps + 1 mma warp

template <int BITS, int PER, int SW>
__global__ void __launch_bounds__(kGemmThreads, 1) nint_gemm_tc_kernel(const GemmArgs a) {
    constexpr int G = kChunkGroups, HALF = PER / 2, GS = 4 * PER, KST = G * GS, ATOMS = KST / 64;
    static_assert(KST % 64 == 0, "a chunk must be whole 64-element swizzle atoms");
    using QU = PairUnit<BITS>;
    using SU = PairUnit<SW>;
    constexpr int WC = QU::words_for(G * PER), SWC = SU::words_for(16), REC = WC * 32 + SWC * 8;
    const NintDev& w = a.w;
    const int BN = a.bn;

    extern __shared__ unsigned char smem_raw[];
    // 1024-byte aligned tile area
    unsigned char* tiles = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    const int a_stage_bytes = ATOMS * 128 * 128, b_stage_bytes = ATOMS * BN * 128;
    unsigned char* a_tile[2] = {tiles, tiles + a_stage_bytes};
    unsigned char* b_tile[2] = {tiles + 2 * a_stage_bytes, tiles + 2 * a_stage_bytes + b_stage_bytes};
    __shared__ __align__(8) uint64_t full_bar[2], empty_bar[2], done_bar;
    __shared__ uint32_t tmem_base_slot;
    __shared__ int failed;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int q = lane >> 2, c = lane & 3;
    const int row0 = blockIdx.x * 128, tok0 = blockIdx.y * BN;

    if (tid == 0) {
        mbar_init(&full_bar[0], 256);
        mbar_init(&full_bar[1], 256);
        mbar_init(&empty_bar[0], 1);
        mbar_init(&empty_bar[1], 1);
        mbar_init(&done_bar, 1);
        failed = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 8) tmem_alloc(&tmem_base_slot, (uint32_t)BN);
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_d = tmem_base_slot;

    if (warp < 8) {
        // ------------------------------ producers ------------------------------
        const int rb = blockIdx.x * 8 + warp;            // row-block of w this warp dequantises
        const bool rb_valid = rb < w.nrb;
        for (int ch = 0; ch < w.nchunks; ++ch) {
            const int st = ch & 1, use = ch >> 1;
            if (use > 0 && !mbar_wait(&empty_bar[st], (use - 1) & 1)) { failed = 1; break; }
            // x slice: BN rows x KST columns, 16-byte chunks, swizzled
            unsigned char* bt = b_tile[st];
            const int chunks_per_row = KST / 8;
            for (int i = tid; i < BN * chunks_per_row; i += 256) {
                const int t = i / chunks_per_row, c16 = i % chunks_per_row;
                const int atom = c16 >> 3, in_atom = c16 & 7;
                unsigned char* dst = bt + atom * (BN * 128) + t * 128 + ((in_atom ^ (t & 7)) << 4);
                const int k0 = ch * KST + c16 * 8, tok = tok0 + t;
                if (tok < a.m && k0 < a.kx) cp_async16(dst, a.x16 + (size_t)tok * a.kx + k0);
                else *reinterpret_cast<uint4*>(dst) = make_uint4(0u, 0u, 0u, 0u);
            }
            cp_async_commit();
            // weight record -> f16 rows of the A tile
            unsigned char* at = a_tile[st];
            if (rb_valid) {
                const uint32_t* rec = w.items + ((size_t)rb * w.nchunks + ch) * REC;
                uint32_t qw[WC], sw[SWC];
#pragma unroll
                for (int j = 0; j < WC; ++j) qw[j] = __ldg(rec + j * 32 + lane);
#pragma unroll
                for (int j = 0; j < SWC; ++j) sw[j] = __ldg(rec + WC * 32 + j * 8 + q);
                const uint32_t an_lo = __ldg(w.anchors + rb * 16 + q), an_hi = __ldg(w.anchors + rb * 16 + 8 + q);
                const float2 f_lo = __half22float2(*reinterpret_cast<const __half2*>(&an_lo));   // (ns, nm)
                const float2 f_hi = __half22float2(*reinterpret_cast<const __half2*>(&an_hi));
                float smin[2][G];
#pragma unroll
                for (int r = 0; r < 2; ++r)
#pragma unroll
                    for (int j = 0; j < 4; ++j) pair_to_floats<SW>(SU::at(sw, 8 + 4 * r + j), smin[r][2 * j], smin[r][2 * j + 1]);
#pragma unroll
                for (int g = 0; g < G; ++g) {
                    float s_lo, s_hi;
                    pair_to_floats<SW>(SU::at(sw, g), s_lo, s_hi);
                    const float d[2] = {f_lo.x * s_lo, f_hi.x * s_hi};
                    const float mn[2] = {f_lo.y * smin[0][g], f_hi.y * smin[1][g]};
#pragma unroll
                    for (int r = 0; r < 2; ++r) {
                        const int row = warp * 16 + q + 8 * r;
#pragma unroll
                        for (int j = 0; j < HALF; ++j) {
                            const uint32_t raw = QU::at(qw, (g * 2 + r) * HALF + j);
                            const float v0 = fmaf(d[r], (float)(raw & 0xFFFFu), -mn[r]);
                            const float v1 = fmaf(d[r], (float)(raw >> 16), -mn[r]);
                            const __half2 h = __floats2half2_rn(v0, v1);
                            const int k = g * GS + c * PER + 2 * j, atom = k >> 6, kk = k & 63;
                            *reinterpret_cast<__half2*>(at + atom * (128 * 128) + row * 128 + (((kk >> 3) ^ q) << 4) + (kk & 7) * 2) = h;
                        }
                    }
                }
            } else {
                // rows past the end of w: zero the warp's 16 rows
                for (int i = lane; i < 16 * ATOMS * 8; i += 32) {
                    const int r = i / (ATOMS * 8), rest = i % (ATOMS * 8), atom = rest >> 3, c16 = rest & 7;
                    *reinterpret_cast<uint4*>(at + atom * (128 * 128) + (warp * 16 + r) * 128 + (c16 << 4)) = make_uint4(0u, 0u, 0u, 0u);
                }
            }
            asm volatile("cp.async.wait_group 0;\n" ::: "memory");
            fence_proxy_async_smem();
            mbar_arrive(&full_bar[st]);
        }
    } else if (lane == 0) {
        // ------------------------------ mma issuer ------------------------------
        const uint32_t idesc = instr_desc_f16(128, BN);
        for (int ch = 0; ch < w.nchunks; ++ch) {
            const int st = ch & 1, use = ch >> 1;
            if (!mbar_wait(&full_bar[st], use & 1)) { failed = 1; break; }
            tc_fence_after_sync();
            const uint32_t a_base = smem_u32(a_tile[st]), b_base = smem_u32(b_tile[st]);
#pragma unroll 1
            for (int j = 0; j < KST / 16; ++j) {
                const uint64_t ad = smem_desc_sw128(a_base + (j >> 2) * (128 * 128) + (j & 3) * 32);
                const uint64_t bd = smem_desc_sw128(b_base + (j >> 2) * (BN * 128) + (j & 3) * 32);
                tc_mma_f16(tmem_d, ad, bd, idesc, ch > 0 || j > 0);
            }
            tc_commit(&empty_bar[st]);
        }
        tc_commit(&done_bar);
    }

    // ------------------------------ epilogue ------------------------------
    if (warp < 8) {
        bool ok = !failed && mbar_wait(&done_bar, 0);
        ok = __all_sync(0xffffffffu, ok);   // tcgen05.ld is warp-wide: take the decision together
        if (!ok) failed = 1;
        tc_fence_after_sync();
        if (ok) {
            const int lane_quarter = warp & 3, col_half = warp >> 2;
            const int n = row0 + lane_quarter * 32 + lane;
            for (int cb = col_half * (BN / 2); cb < (col_half + 1) * (BN / 2); cb += 32) {
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
    if (warp == 8) {
        tmem_free(tmem_d, (uint32_t)BN);
        if (lane == 0 && failed) atomicExch(a.error, MFQB_ERR_TIMEOUT);
    }
}

struct GemmPlan {
    int bn, grid_x, grid_y;
    size_t smem;
};
// gs must be 16, 24 or 32 (a chunk is then whole swizzle atoms); returns bn = 0 otherwise.
inline GemmPlan plan_nint_gemm(const NintDev& w, int m) {
    GemmPlan p{};
    if (!(w.gs == 16 || w.gs == 24 || w.gs == 32) || w.per * 4 != w.gs) return p;
    const int kst = kChunkGroups * w.gs, atoms = kst / 64;
    int bn = w.gs == 16 ? 256 : (w.gs == 24 ? 128 : 64);
    while (bn > 64 && bn / 2 >= m) bn /= 2;
    p.bn = bn;
    p.grid_x = (w.n + 127) / 128;
    p.grid_y = (m + bn - 1) / bn;
    p.smem = (size_t)2 * atoms * (128 + bn) * 128 + 1024;
    return p;
}

template <int BITS>
cudaError_t launch_nint_gemm_bits(const GemmArgs& a, const GemmPlan& p, cudaStream_t stream);

}  // namespace mfqb
