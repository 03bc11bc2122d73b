// Prefill GEMM for NINT weights on tcgen05 tensor cores with the accumulator in tensor memory.
//
//   y[m, n] = sum_k x[m, k] * W[n, k]           (m = tokens, large;  W packed NINT)
//
// One CTA owns a tile of 128 weight rows x BN tokens and walks K one chunk (8 groups) at a time
// through a two-stage shared-memory ring:
//   * 16 producer warps: a pair of warps dequantises the chunk's record of one row-block of the
//     tile (w = d*q - m in float32, rounded once to f16) into the A atoms; one more warp feeds the
//     BN x 64 slices of x (f16) into the B atoms with TMA; both are K-major rows of 128 bytes with
//     the 128-byte swizzle the tensor core expects;
//   * one warp: one thread issues tcgen05.mma (M = 128, N = BN, K = 16 per instruction) for the
//     chunk, D accumulating in tensor memory, and tcgen05.commit hands the stage back;
//   * epilogue: the producer warps read the accumulator with tcgen05.ld (lane = weight row) and store y.
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

#include "nint_gemv1_bl.cuh"
#include "tc05.cuh"

namespace mfqb {

struct GemmArgs {
    NintDevB w;
    const __half* x16;   // [m, kx] f16, kx = k rounded up to 8, zero padded
    int m, kx;
    void* y;             // [m, n]
    int y_dtype;
    int bn;              // tokens per tile: 64, 128, 256 or 512
    int stages;          // depth of the weight ring, in 64-column atoms (at least one chunk)
    int xstages;         // depth of the activation ring, in stages of xcols columns
    int xcols;           // columns of K per activation stage: 64 (128-byte rows, 128-byte swizzle) or 32 (64-byte rows, 64-byte swizzle)
    int* error;          // device word: set to MFQB_ERR_TIMEOUT when a wait expires
    // Grouped mode (expert matmul over a route plan whose tile size is bn): blockIdx.y is a tile of
    // up to bn pairs of one expert; x16 holds the input rows in plan order (row p = pair
    // pair_order[p]), the tile's expert selects rb_per_expert row-blocks of w, and the result of
    // column i goes to row pair_order[p0 + i] of y [pairs, ldy].  tile_bounds == nullptr: plain GEMM.
    const int* expert_bounds;
    const int* tile_bounds;
    const int* pair_order;
    const int* expert_pool;
    const int* expert_local;
    int n_experts, pool, rb_per_expert, ldy;
};

constexpr int kGemmProducerWarps = 16;
// The f16 weights carry a factor 2^10 (taken out of the accumulators in the epilogue): f16 keeps all its bits for
// quantisation steps down to 2^-24 and represents weights up to 64.
constexpr float kGemmWeightScale = 1024.f, kGemmWeightUndo = 1.f / 1024.f;
constexpr int kGemmThreads = (kGemmProducerWarps + 2) * 32;   // + mma warp + x loader warp

// Two rings, both counted in atoms of 64 columns of K, each atom a K-major tile with the 128-byte
// swizzle: the weight ring holds 128 x 64 f16 slabs of W (16 KB; a chunk of 8 groups is ATOMS
// consecutive stages and is decoded as a whole, so the ring holds at least one chunk), the
// activation ring BN x 64 f16 slabs of x, which only need to run a little ahead of the tensor core.  Two producer warps share one row-block record: warp half f decodes
// the registers of family f (groups 4f .. 4f+3) of the byte-lane layout.
template <int BITS, int T>
__global__ void __launch_bounds__(kGemmThreads, 1) nint_gemm_tc_kernel(const GemmArgs a, const __grid_constant__ CUtensorMap x_map) {
    constexpr int G = kChunkGroupsB, GS = 8 * T, KST = G * GS, ATOMS = KST / 64;
    static_assert(KST % 64 == 0, "a chunk must be whole 64-element swizzle atoms");
    using BU = ByteUnit<BITS>;
    constexpr int WC = BU::words_for(8 * T), REC = (WC + 2) * 32;
    // words of one family: registers [f * 4T, (f + 1) * 4T) start on a unit boundary when 4T is a
    // multiple of the unit's register count; otherwise the warp reads the whole stream
    constexpr bool SPLIT = (4 * T) % BU::NP == 0;
    constexpr int FW = SPLIT ? (4 * T) / BU::NP * BU::U : WC;
    constexpr int NPROD = kGemmProducerWarps * 32;
    const NintDevB& w = a.w;
    const int BN = a.bn, NS = a.stages, NB = a.xstages;

    extern __shared__ unsigned char smem_raw[];
    unsigned char* tiles = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    constexpr int stage_bytes = 128 * 128;           // one weight atom
    const int XC = a.xcols, xper = 64 / XC;          // activation stages per weight atom
    const int xstage_bytes = BN * XC * 2;            // one activation stage
    unsigned char* xtiles = tiles + (size_t)NS * stage_bytes;
    __shared__ __align__(8) uint64_t full_bar[8], empty_bar[8], xfull_bar[4], xempty_bar[4], done_bar;
    __shared__ uint32_t tmem_base_slot;
    __shared__ int failed;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int q = lane >> 2, c = lane & 3;
    int row0 = blockIdx.x * 128, tok0 = blockIdx.y * BN;
    int rb_first = blockIdx.x * 8, rb_end = w.nrb, ncols = a.m - tok0, row_limit = w.n, ldy = w.n;
    const bool grouped = a.tile_bounds != nullptr;
    if (grouped) {
        const int t = blockIdx.y;
        if (t >= a.tile_bounds[a.n_experts]) return;   // before any barrier or tensor-memory allocation: the whole CTA leaves
        int lo = 0, hi = a.n_experts - 1;   // expert e with tile_bounds[e] <= t < tile_bounds[e + 1]
        while (lo < hi) {
            const int mid = (lo + hi + 1) >> 1;
            if (a.tile_bounds[mid] <= t) lo = mid;
            else hi = mid - 1;
        }
        if (a.expert_pool[lo] != a.pool) return;
        tok0 = a.expert_bounds[lo] + (t - a.tile_bounds[lo]) * BN;
        ncols = a.expert_bounds[lo + 1] - tok0;
        const int rb_base = a.expert_local[lo] * a.rb_per_expert;
        rb_first = rb_base + blockIdx.x * 8;
        rb_end = rb_base + a.rb_per_expert;
        row_limit = a.ldy;   // rows of one expert
        ldy = a.ldy;
    }
    if (ncols > BN) ncols = BN;

    if (tid == 0) {
        for (int i = 0; i < 8; ++i) {
            mbar_init(&full_bar[i], NPROD);
            mbar_init(&empty_bar[i], 1);
        }
        for (int i = 0; i < 4; ++i) {
            mbar_init(&xfull_bar[i], 1);   // the x loader's expect_tx arrival
            mbar_init(&xempty_bar[i], 1);
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
        const int rbl = warp >> 1, f = warp & 1;         // row-block of the tile, family of the chunk
        const int rb = rb_first + rbl;
        const bool rb_valid = rb < rb_end;
        bool alive = true;
        const int w0 = SPLIT ? f * FW : 0;               // first code word of this warp's registers
        const int r0 = SPLIT ? 0 : f * 4 * T;            // register index of (t = 0, a = 0) inside those words
        uint32_t nq[FW], nsc[4];
        auto fetch = [&](int ch) {
            const uint32_t* rec = w.items + ((size_t)rb * w.nchunks + ch) * REC;
#pragma unroll
            for (int j = 0; j < FW; ++j) nq[j] = __ldg(rec + (w0 + j) * 32 + lane);
            // scale words of the lanes that own (rows q, q+8) x groups 4f + {0,1} and 4f + {2,3}
#pragma unroll
            for (int j = 0; j < 4; ++j) nsc[j] = __ldg(rec + (WC + (j >> 1)) * 32 + 4 * q + 2 * f + (j & 1));
        };
        if (rb_valid) fetch(0);
        // where each of the lane's registers of a chunk goes: atom (k / 64) and swizzled byte offset inside the atom
        uint32_t slot_of[4 * T];
#pragma unroll
        for (int t = 0; t < T; ++t)
#pragma unroll
            for (int aa = 0; aa < 4; ++aa) {
                const int row = rbl * 16 + q + 8 * (aa & 1);
                const int k = (4 * f + 2 * (aa >> 1) + (c >> 1)) * GS + 8 * t + 4 * (c & 1), atom = k >> 6, kk = k & 63;
                slot_of[t * 4 + aa] = ((uint32_t)atom << 14) | (uint32_t)(row * 128 + (((kk >> 3) ^ q) << 4) + (kk & 7) * 2);
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
                uint32_t qw[FW], sc[4];
#pragma unroll
                for (int j = 0; j < FW; ++j) qw[j] = nq[j];
#pragma unroll
                for (int j = 0; j < 4; ++j) sc[j] = nsc[j];
                if (ch + 1 < w.nchunks) fetch(ch + 1);   // next record's words are requested before this one is decoded
                const uint32_t an_lo = __ldg(w.anchors + rb * 16 + q), an_hi = __ldg(w.anchors + rb * 16 + 8 + q);
                const float2 f_lo = __half22float2(*reinterpret_cast<const __half2*>(&an_lo));   // (ns, nm)
                const float2 f_hi = __half22float2(*reinterpret_cast<const __half2*>(&an_hi));
                // register a of a step: row q + 8(a&1), group 4f + 2(a>>1) + (c>>1); its scale bytes sit in
                // word (a>>1) of the pair fetched above, byte 2(a&1) + (c>>1).  The weight is built in f16:
                // d' (q - q_mid) + n' with d' = 2^10 d and n' = -(2^10 m - d' q_mid) rounded to f16 (the factor
                // 2^10 keeps small quantisation steps normal numbers; the epilogue takes it out again).
                __half2 d2[4], n2[4];
#pragma unroll
                for (int aa = 0; aa < 4; ++aa) {
                    const int sh = 8 * (2 * (aa & 1) + (c >> 1));
                    const float ss = (float)((sc[aa >> 1] >> sh) & 0xFF), sm = (float)((sc[2 + (aa >> 1)] >> sh) & 0xFF);
                    const float dd = kGemmWeightScale * ((aa & 1) ? f_hi.x : f_lo.x) * ss;
                    d2[aa] = __float2half2_rn(dd);
                    n2[aa] = __float2half2_rn(fmaf(dd, (float)(1 << (BITS - 1)), -kGemmWeightScale * ((aa & 1) ? f_hi.y : f_lo.y) * sm));
                }
                const __half2 bias = __float2half2_rn(1024.f + (float)(1 << (BITS - 1)));
                const int st_base = (ch * ATOMS) % NS;
#pragma unroll
                for (int t = 0; t < T; ++t) {
#pragma unroll
                    for (int aa = 0; aa < 4; ++aa) {
                        const uint32_t v = BU::at(qw, r0 + t * 4 + aa);
                        // a code byte under the exponent byte 0x64 is the f16 1024 + q
                        const uint32_t lo = __byte_perm(v, 0x64646464u, 0x4140), hi = __byte_perm(v, 0x64646464u, 0x4342);
                        const __half2 h01 = __hfma2(__hsub2(*reinterpret_cast<const __half2*>(&lo), bias), d2[aa], n2[aa]);
                        const __half2 h23 = __hfma2(__hsub2(*reinterpret_cast<const __half2*>(&hi), bias), d2[aa], n2[aa]);
                        const uint32_t pk = slot_of[t * 4 + aa];   // atom of the chunk (high bits) and byte offset inside it, fixed per lane
                        int st = st_base + (int)(pk >> 14);
                        if (st >= NS) st -= NS;
                        uint2 out;
                        out.x = *reinterpret_cast<const uint32_t*>(&h01);
                        out.y = *reinterpret_cast<const uint32_t*>(&h23);
                        *reinterpret_cast<uint2*>(tiles + st * stage_bytes + (pk & 0x3FFFu)) = out;
                    }
                }
            } else if (f == 0) {
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
            const int nx = w.nchunks * ATOMS * xper;
            for (int xi = 0; xi < nx; ++xi) {
                const int st = xi % NB, use = xi / NB;
                if (use > 0 && !mbar_wait(&xempty_bar[st], (use - 1) & 1)) { failed = 1; break; }
                mbar_arrive_expect_tx(&xfull_bar[st], (uint32_t)xstage_bytes);
                for (int r0 = 0; r0 < BN; r0 += 256)   // a box holds at most 256 rows
                    tma_load_2d(xtiles + (size_t)st * xstage_bytes + (size_t)r0 * XC * 2, &x_map, xi * XC, tok0 + r0, &xfull_bar[st]);
            }
        }
    } else if (lane == 0) {
        // ------------------------------ mma issuer ------------------------------
        const uint32_t idesc = instr_desc_f16(128, BN < 256 ? BN : 256);
        const int natoms = w.nchunks * ATOMS;
        if (XC == 64) {   // one activation stage per weight atom
            for (int ai = 0; ai < natoms; ++ai) {
                const int st = ai % NS, xs = ai % NB;
                if (!mbar_wait(&full_bar[st], (ai / NS) & 1) || !mbar_wait(&xfull_bar[xs], (ai / NB) & 1)) { failed = 1; break; }
                tc_fence_after_sync();
                const uint32_t a_base = smem_u32(tiles + st * stage_bytes), b_base = smem_u32(xtiles + (size_t)xs * xstage_bytes);
#pragma unroll
                for (int j = 0; j < 4; ++j)
                    for (int h = 0; h < BN; h += 256)   // one instruction covers at most 256 token columns
                        tc_mma_f16(tmem_d + (uint32_t)h, smem_desc_sw128(a_base + j * 32), smem_desc_sw128(b_base + h * 128 + j * 32), idesc,
                                   ai > 0 || j > 0);
                tc_commit(&empty_bar[st]);
                tc_commit(&xempty_bar[xs]);
            }
        } else {          // two 32-column activation stages (64-byte rows) per weight atom
            bool ok = true;
            for (int ai = 0; ai < natoms && ok; ++ai) {
                const int st = ai % NS;
                if (!mbar_wait(&full_bar[st], (ai / NS) & 1)) { failed = 1; break; }
                const uint32_t a_base = smem_u32(tiles + st * stage_bytes);
#pragma unroll
                for (int xh = 0; xh < 2; ++xh) {
                    const int xi = ai * 2 + xh, xs = xi % NB;
                    if (!mbar_wait(&xfull_bar[xs], (xi / NB) & 1)) { failed = 1; ok = false; break; }
                    tc_fence_after_sync();
                    const uint32_t b_base = smem_u32(xtiles + (size_t)xs * xstage_bytes);
#pragma unroll
                    for (int jj = 0; jj < 2; ++jj)
                        for (int h = 0; h < BN; h += 256)
                            tc_mma_f16(tmem_d + (uint32_t)h, smem_desc_sw128(a_base + (xh * 2 + jj) * 32), smem_desc_sw64(b_base + h * 64 + jj * 32), idesc,
                                       ai > 0 || xh > 0 || jj > 0);
                    tc_commit(&xempty_bar[xs]);
                }
                if (ok) tc_commit(&empty_bar[st]);
            }
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
            const int n = row0 + lane_quarter * 32 + lane;   // row of the matrix, or of the tile's expert
            for (int cb = c_begin; cb < c_end; cb += 32) {
                uint32_t r[32];
                tmem_ld32(tmem_d + ((uint32_t)(lane_quarter * 32) << 16) + (uint32_t)cb, r);
                if (n < row_limit) {
#pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        if (cb + i < ncols) {
                            const size_t out_row = grouped ? (size_t)a.pair_order[tok0 + cb + i] : (size_t)(tok0 + cb + i);
                            const float v = __uint_as_float(r[i]) * kGemmWeightUndo;
                            if (a.y_dtype == 0 /* MFQB_F32 */) reinterpret_cast<float*>(a.y)[out_row * ldy + n] = v;
                            else reinterpret_cast<__nv_bfloat16*>(a.y)[out_row * ldy + n] = __float2bfloat16_rn(v);
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

// Dynamic shared memory a tile kernel may plan with: 227 KB per CTA less the alignment slack and the barriers.
constexpr size_t kGemmSmemBudget = 227 * 1024 - 1024 - 512;
// Measurement switch (mfqb_tune "gemm_plan"): 0 = by shape, 1 = 32-column activation stages and a two-chunk weight ring.
extern int g_gemm_plan_choice;
struct GemmPlan {
    int bn, stages, xstages, xcols, grid_x, grid_y;
    size_t smem;
};
// The group size must be a multiple of 8 (a chunk is then whole swizzle atoms); returns bn = 0 otherwise.
inline GemmPlan plan_nint_gemm(const NintDevB& w, int m) {
    GemmPlan p{};
    if (w.gs % 8 != 0 || w.t8 * 8 != w.gs) return p;
    const int atoms = kChunkGroupsB * w.gs / 64;
    // 512-token tiles amortise the dequantisation best.  With two 64-column activation stages (128 KB) the
    // weight ring holds five atoms: one whole chunk of up to four atoms, whose decode then overlaps the
    // tensor core only a little.  Measured, that still beats a two-chunk weight ring
    // fed by three 32-column stages (424 against 578 TFLOP/s for group size 32): every stage is a
    // separate trip to L2, and the tile's activation feed -- 64 bytes per clock per SM at the tensor
    // core's full rate -- is what bounds the kernel.  The 32-column stages remain for chunks that
    // would not fit otherwise.
    auto stages_for = [](int bn_, int xcols, int xst) { return std::min(8, (int)((kGemmSmemBudget - (size_t)xst * bn_ * xcols * 2) / (128 * 128))); };
    int bn = 512, xcols = 64, xst = 2;
    if (atoms > 5 || g_gemm_plan_choice == 1) {   // (a six-atom chunk fits beside two 64-column stages, but measured slower than the 32-column form)
        if (stages_for(512, 32, 3) >= atoms) { xcols = 32; xst = 3; }
        else {
            bn = 256;
            xst = 3;
            while (bn > 128 && stages_for(bn, 64, 3) < atoms) bn /= 2;
        }
    }
    while (bn > 64 && bn / 2 >= m) {
        bn /= 2;
        xcols = 64;
        xst = 3;
    }
    p.bn = bn;
    p.xstages = xst;
    p.xcols = xcols;
    p.stages = stages_for(bn, xcols, xst);
    if (bn == 512 && xcols == 64) p.stages = std::min(p.stages, 5);   // five beat six (578 against 505 TFLOP/s on 14336 x 4096, 512 tokens)
    if (p.stages < atoms) { p.bn = 0; return p; }
    p.grid_x = (w.n + 127) / 128;
    p.grid_y = (m + bn - 1) / bn;
    p.smem = (size_t)p.stages * 128 * 128 + (size_t)p.xstages * bn * p.xcols * 2 + 1024;
    return p;
}

// Plan of the grouped mode for a fixed token tile (the route plan's tile size, 32 .. 256); grid_x
// covers one expert's rows.  bn = 0 when this weight has no tile kernel for it.
inline GemmPlan plan_nint_gemm_grouped(const NintDevB& w, int bn, int rows_per_expert, int max_tiles) {
    GemmPlan p{};
    if (w.gs % 8 != 0 || w.t8 * 8 != w.gs || bn < 32 || bn > 256 || (bn & (bn - 1))) return p;
    const int atoms = kChunkGroupsB * w.gs / 64;
    p.bn = bn;
    p.xstages = 3;
    p.xcols = 64;
    p.stages = std::min(8, (int)((kGemmSmemBudget - (size_t)p.xstages * bn * 128) / (128 * 128)));
    if (p.stages < atoms) { p.bn = 0; return p; }
    p.grid_x = (rows_per_expert + 127) / 128;
    p.grid_y = max_tiles;
    p.smem = (size_t)p.stages * 128 * 128 + (size_t)p.xstages * bn * 128 + 1024;
    return p;
}

template <int BITS>
cudaError_t launch_nint_gemm_bits(const GemmArgs& a, const GemmPlan& p, const CUtensorMap& x_map, cudaStream_t stream);

template <int BITS, int T>
static cudaError_t launch_nint_gemm_one(const GemmArgs& a, const GemmPlan& p, const CUtensorMap& x_map, cudaStream_t stream) {
    if constexpr (nint_bl_in_catalog(BITS, T)) {
        auto kern = nint_gemm_tc_kernel<BITS, T>;
        const cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)p.smem);
        if (e != cudaSuccess) return e;
        kern<<<dim3((unsigned)p.grid_x, (unsigned)p.grid_y), kGemmThreads, p.smem, stream>>>(a, x_map);
        return cudaGetLastError();
    } else {
        return cudaErrorNotSupported;
    }
}

// One translation unit per code width (nint_gemm_b*.cu) instantiates the launch table.
#define MFQB_GEMM_INSTANTIATE(BITS)                                                                                                     \
    template <>                                                                                                                         \
    cudaError_t launch_nint_gemm_bits<BITS>(const GemmArgs& a, const GemmPlan& p, const CUtensorMap& x_map, cudaStream_t stream) {      \
        switch (a.w.t8) {                                                                                                               \
            case 2: return launch_nint_gemm_one<BITS, 2>(a, p, x_map, stream);                                                          \
            case 3: return launch_nint_gemm_one<BITS, 3>(a, p, x_map, stream);                                                          \
            case 4: return launch_nint_gemm_one<BITS, 4>(a, p, x_map, stream);                                                          \
            case 5: return launch_nint_gemm_one<BITS, 5>(a, p, x_map, stream);                                                          \
            case 6: return launch_nint_gemm_one<BITS, 6>(a, p, x_map, stream);                                                          \
            case 8: return launch_nint_gemm_one<BITS, 8>(a, p, x_map, stream);                                                          \
            default: return cudaErrorNotSupported;                                                                                      \
        }                                                                                                                               \
    }

}  // namespace mfqb
