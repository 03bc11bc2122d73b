// Single-row (m = 1) GEMV for NINT weights: the decode hot path.
//
// With one activation row the n8 slot of the tensor-core tile is free, so the eight columns
// carry the eight *groups* of a chunk instead of batch rows: the B operand is block-diagonal
// (column g holds x only at the k-slots that belong to group g), and one accumulator tile
// D[16 rows][8 groups] collects  sum_{k in g} (128 + q) x  for all groups of the chunk at once.
// The per-group integer sub-scales and sub-mins are then applied once per chunk -- lane (q, c)
// owns groups 2c, 2c+1 of rows q, q+8, so nothing is decoded twice -- and a quad reduction
// adds the eight groups.  Every mma handles pair j of group g (slots 2c, 2c+1) and of group
// g+4 (slots 2c+8, 2c+9), which the lane-stream layout already provides.
// The group sums of x (for the -128 seed and the sub-min term) are computed once per CTA into a
// shared-memory table while x is staged.
#pragma once
#include "nint_gemv.cuh"

namespace mfqb {

__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gsrc) {
    const unsigned d = (unsigned)__cvta_generic_to_shared(smem_dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(d), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
// Records per warp ring: about 6 KB of ring per warp (three 8-warp CTAs per SM then keep well
// over 100 KB of weight bytes requested per SM), between 2 and 6 stages.
__host__ __device__ constexpr int gemv_m1_stages(int rec_words) {
    return 6144 / (rec_words * 4) < 2 ? 2 : (6144 / (rec_words * 4) > 6 ? 6 : 6144 / (rec_words * 4));
}

// Shared memory: partial sums [rb_per_cta][16] f32 | anchors [rb_per_cta][16] u32 | x bf16
// [xstride] | per warp a ring of `stages` item records.  Every warp streams its own items
// (chunk-major, as in the batched kernel) through its ring with 16-byte asynchronous copies:
// nothing a copy in flight occupies is a register, so a CTA keeps tens of kilobytes requested
// at all times; the first `stages` items are requested before the kernel waits for its
// predecessor in the stream, since weights are constants.
template <int BITS, int PER, int SW>
__global__ void __launch_bounds__(256, 3) nint_gemv_m1_kernel(const GemvArgs a) {
    constexpr int G = kChunkGroups, HALF = PER / 2;
    constexpr int NPL = BITS == 8 ? 2 : 1;
    static_assert(G == 8, "eight groups per chunk map onto the eight mma columns");
    using QU = PairUnit<BITS>;
    using SU = PairUnit<SW>;
    constexpr int WC = QU::words_for(G * PER), SWC = SU::words_for(16), REC = WC * 32 + SWC * 8;
    constexpr int S = gemv_m1_stages(REC);
    const NintDev& w = a.w;

    extern __shared__ __align__(16) unsigned char smem[];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarps = blockDim.x >> 5;
    const int q = lane >> 2, c = lane & 3;
    float* ypart = reinterpret_cast<float*>(smem);
    uint32_t* anch = reinterpret_cast<uint32_t*>(ypart + (size_t)a.rb_per_cta * 16);
    __nv_bfloat16* xs = reinterpret_cast<__nv_bfloat16*>(anch + (size_t)a.rb_per_cta * 16);
    float* xsum_tab = reinterpret_cast<float*>(xs + a.xstride);            // [nchunks * 8] group sums of x
    uint32_t* ring = reinterpret_cast<uint32_t*>(xsum_tab + w.nchunks * G) + (size_t)warp * S * REC;
    // balanced split of the row-blocks over gridDim.x: CTA b owns [b*R/grid, (b+1)*R/grid) of the
    // R row-blocks of the whole matrix, or of its pair's expert in routed mode
    int rb_base = 0, rb_total = w.nrb;
    const __nv_bfloat16* xrow = a.x;
    size_t y_off = 0;
    if (a.route_ids != nullptr) {
        pdl_wait();   // the routing table comes from the previous kernel
        const int pair = blockIdx.y, e = a.route_ids[pair];
        if (e < 0 || a.expert_pool[e] != a.pool) return;
        rb_total = a.rb_per_expert;
        rb_base = a.expert_local[e] * a.rb_per_expert;
        xrow += (size_t)(a.x_per_pair ? pair : pair / a.routes) * w.k;
        y_off = (size_t)pair * a.ldy;
    }
    const int rbl0 = (int)(((long long)blockIdx.x * rb_total) / gridDim.x);
    const int nrb = (int)(((long long)(blockIdx.x + 1) * rb_total) / gridDim.x) - rbl0;
    const int rb0 = rb_base + rbl0;
    const int row_limit = a.route_ids != nullptr ? a.ldy : w.n;   // rows this problem has (an expert's rows are padded to whole blocks)

    // items of this warp, chunk-major: chunk = warp, warp + nwarps, ...; inside a chunk every
    // row-block of the CTA.  Two cursors walk that sequence (issue runs S items ahead); they are
    // advanced incrementally -- no division in the loop.
    const int my_segs = warp < w.nchunks ? (w.nchunks - warp + nwarps - 1) / nwarps : 0;
    const int n_mine = a.stages == -1 ? 0 : my_segs * nrb;
    int iss_i = 0, iss_seg = warp, iss_rbl = 0, iss_stage = 0;
    auto issue = [&]() {
        if (iss_i < n_mine) {
            const uint32_t* src = w.items + ((size_t)(rb0 + iss_rbl) * w.nchunks + iss_seg) * REC;
            uint32_t* dst = ring + iss_stage * REC;
#pragma unroll
            for (int off = 0; off < REC; off += 128)
                if (off + 128 <= REC || lane * 4 < REC - off) cp_async16(dst + off + lane * 4, src + off + lane * 4);
        }
        cp_async_commit();   // one group per item slot, empty past the end: keeps the wait count uniform
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
    pdl_wait();
    {   // stage x (zero beyond k): 16-byte copies when the row is 16-byte aligned
        const int kp = a.xstride;
        if ((w.k & 7) == 0 && (reinterpret_cast<uintptr_t>(xrow) & 15) == 0) {
            for (int v = tid; v < kp / 8; v += blockDim.x) {
                uint4 val = make_uint4(0u, 0u, 0u, 0u);
                if (v * 8 < w.k) val = __ldg(reinterpret_cast<const uint4*>(xrow) + v);
                *reinterpret_cast<uint4*>(xs + v * 8) = val;
            }
        } else {
            for (int k = tid; k < kp; k += blockDim.x) xs[k] = k < w.k ? xrow[k] : __float2bfloat16(0.f);
        }
    }
    __syncthreads();
    const uint32_t* xw = reinterpret_cast<const uint32_t*>(xs);
    // group sums of x, once per CTA: seed of the accumulators (-128 * sum) and the sub-min term
    for (int g = tid; g < w.nchunks * G; g += blockDim.x) {
        float s = 0.f;
        const uint32_t* p = xw + (g * w.gs) / 2;
        for (int e = 0; e < w.gs / 2; ++e) {
            const uint32_t v = p[e];
            s += __uint_as_float(v << 16) + __uint_as_float(v & 0xFFFF0000u);
        }
        xsum_tab[g] = s;
    }
    __syncthreads();
    int cur_seg = -1;
    uint32_t b0[4][HALF], b1[4][HALF];   // block-diagonal B: non-zero only where the lane's column is the mma's group
    float xs0 = 0.f, xs1 = 0.f;          // group sums of x for groups 2c, 2c+1 of the chunk

    auto prepare_chunk = [&](int seg) {
        uint32_t xq[HALF];
#pragma unroll
        for (int j = 0; j < HALF; ++j) {
            // slots past the group width (padded PER) carry zero codes; they must not read x at all:
            // on the last group the index would run past the staged row
            xq[j] = 0u;
            if (c * PER + 2 * j < w.gs) xq[j] = xw[((seg * G + q) * w.gs + c * PER) / 2 + j];
        }
#pragma unroll
        for (int g = 0; g < 4; ++g) {
#pragma unroll
            for (int j = 0; j < HALF; ++j) {
                b0[g][j] = q == g ? xq[j] : 0u;
                b1[g][j] = q == g + 4 ? xq[j] : 0u;
            }
        }
        const float2 sums = *reinterpret_cast<const float2*>(xsum_tab + seg * G + 2 * c);
        xs0 = sums.x;
        xs1 = sums.y;
    };

    int seg = warp, rbl = 0, stage = 0;
    for (int i = 0; i < n_mine; ++i) {
        if (seg != cur_seg) { cur_seg = seg; prepare_chunk(seg); }
        asm volatile("cp.async.wait_group %0;\n" ::"n"(S - 1) : "memory");
        __syncwarp();
        const uint32_t* rec = ring + stage * REC;
        uint32_t qw[WC], sw[SWC];
#pragma unroll
        for (int j = 0; j < WC; ++j) qw[j] = rec[j * 32 + lane];
#pragma unroll
        for (int j = 0; j < SWC; ++j) sw[j] = rec[WC * 32 + j * 8 + q];
        __syncwarp();          // every lane has read the stage before it is refilled
        issue();
        if (a.stages == -2) {   // DBG: memory pipeline only
            uint32_t v = 0;
#pragma unroll
            for (int j = 0; j < WC; ++j) v ^= qw[j];
#pragma unroll
            for (int j = 0; j < SWC; ++j) v ^= sw[j];
            if (v == 0x12345678u) atomicAdd(ypart + rbl * 16 + q, 1.f);
            if (++rbl == nrb) { rbl = 0; seg += nwarps; }
            if (++stage == S) stage = 0;
            continue;
        }

        const float seed0 = (NPL == 2 ? -128.f * 17.f : -128.f) * xs0, seed1 = (NPL == 2 ? -128.f * 17.f : -128.f) * xs1;
        float ch[4][4], hi[2][4];   // chains; hi = high nibbles (8-bit codes); seeds are added at the end
#pragma unroll
        for (int g = 0; g < 4; ++g) {
#pragma unroll
            for (int j = 0; j < HALF; ++j) {
                const uint32_t r0 = QU::at(qw, (g * 2 + 0) * HALF + j), r1 = QU::at(qw, (g * 2 + 1) * HALF + j);
                const uint32_t r2 = QU::at(qw, ((g + 4) * 2 + 0) * HALF + j), r3 = QU::at(qw, ((g + 4) * 2 + 1) * HALF + j);
                if constexpr (NPL == 1) {
                    if (j == 0) mma_k16_first(ch[g], r0 | kBf16x2_128, r1 | kBf16x2_128, r2 | kBf16x2_128, r3 | kBf16x2_128, b0[g][j], b1[g][j]);
                    else mma_k16(ch[g], r0 | kBf16x2_128, r1 | kBf16x2_128, r2 | kBf16x2_128, r3 | kBf16x2_128, b0[g][j], b1[g][j]);
                } else if (g < 2 && j == 0) {
                    constexpr uint32_t NIB = 0x000F000Fu;
                    mma_k16_first(ch[g & 1], (r0 & NIB) | kBf16x2_128, (r1 & NIB) | kBf16x2_128, (r2 & NIB) | kBf16x2_128,
                                  (r3 & NIB) | kBf16x2_128, b0[g][j], b1[g][j]);
                    mma_k16_first(hi[g & 1], ((r0 >> 4) & NIB) | kBf16x2_128, ((r1 >> 4) & NIB) | kBf16x2_128,
                                  ((r2 >> 4) & NIB) | kBf16x2_128, ((r3 >> 4) & NIB) | kBf16x2_128, b0[g][j], b1[g][j]);
                } else {
                    constexpr uint32_t NIB = 0x000F000Fu;
                    mma_k16(ch[g & 1], (r0 & NIB) | kBf16x2_128, (r1 & NIB) | kBf16x2_128, (r2 & NIB) | kBf16x2_128,
                            (r3 & NIB) | kBf16x2_128, b0[g][j], b1[g][j]);
                    mma_k16(hi[g & 1], ((r0 >> 4) & NIB) | kBf16x2_128, ((r1 >> 4) & NIB) | kBf16x2_128,
                            ((r2 >> 4) & NIB) | kBf16x2_128, ((r3 >> 4) & NIB) | kBf16x2_128, b0[g][j], b1[g][j]);
                }
            }
        }
        float acc[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float seed = (e & 1) ? seed1 : seed0;
            if constexpr (NPL == 1) acc[e] = ((ch[0][e] + ch[1][e]) + (ch[2][e] + ch[3][e])) + seed;
            else acc[e] = fmaf(16.f, hi[0][e] + hi[1][e], ch[0][e] + ch[1][e]) + seed;
        }
        // sub-scales / sub-mins of rows (q, q+8) x groups (2c, 2c+1)
        uint32_t sp0, sp1, mp_lo, mp_hi;
        switch (c) {
            case 0: sp0 = SU::at(sw, 0); sp1 = SU::at(sw, 1); mp_lo = SU::at(sw, 8); mp_hi = SU::at(sw, 12); break;
            case 1: sp0 = SU::at(sw, 2); sp1 = SU::at(sw, 3); mp_lo = SU::at(sw, 9); mp_hi = SU::at(sw, 13); break;
            case 2: sp0 = SU::at(sw, 4); sp1 = SU::at(sw, 5); mp_lo = SU::at(sw, 10); mp_hi = SU::at(sw, 14); break;
            default: sp0 = SU::at(sw, 6); sp1 = SU::at(sw, 7); mp_lo = SU::at(sw, 11); mp_hi = SU::at(sw, 15); break;
        }
        float s0_lo, s0_hi, s1_lo, s1_hi, m0_lo, m1_lo, m0_hi, m1_hi;
        pair_to_floats<SW>(sp0, s0_lo, s0_hi);
        pair_to_floats<SW>(sp1, s1_lo, s1_hi);
        pair_to_floats<SW>(mp_lo, m0_lo, m1_lo);
        pair_to_floats<SW>(mp_hi, m0_hi, m1_hi);
        const uint32_t an_lo = anch[rbl * 16 + q], an_hi = anch[rbl * 16 + q + 8];
        const float2 f_lo = __half22float2(*reinterpret_cast<const __half2*>(&an_lo));   // (ns, nm)
        const float2 f_hi = __half22float2(*reinterpret_cast<const __half2*>(&an_hi));
        float v_lo = f_lo.x * fmaf(s1_lo, acc[1], s0_lo * acc[0]) - f_lo.y * fmaf(m1_lo, xs1, m0_lo * xs0);
        float v_hi = f_hi.x * fmaf(s1_hi, acc[3], s0_hi * acc[2]) - f_hi.y * fmaf(m1_hi, xs1, m0_hi * xs0);
        // the four lanes of a quad hold different groups of the same two rows
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
        const int row = rbl0 * 16 + i;   // row inside the problem (matrix, or the pair's expert)
        if (row < row_limit) {
            const float v = ypart[i];
            if (a.y_dtype == 0 /* MFQB_F32 */) reinterpret_cast<float*>(a.y)[y_off + row] = v;
            else reinterpret_cast<__nv_bfloat16*>(a.y)[y_off + row] = __float2bfloat16_rn(v);
        }
    }
}

}  // namespace mfqb
