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
// The group sums of x (for the -128 seed and the sub-min term) come out of the same
// tensor-core pattern with A = 1.
#pragma once
#include "nint_gemv.cuh"

namespace mfqb {

template <int BITS, int PER, int SW>
__global__ void __launch_bounds__(256, 2) nint_gemv_m1_kernel(const GemvArgs a) {
    constexpr int G = kChunkGroups, HALF = PER / 2;
    constexpr int NPL = BITS == 8 ? 2 : 1;
    static_assert(G == 8, "eight groups per chunk map onto the eight mma columns");
    using Item = GemvItem<BITS, PER, SW>;
    using QU = PairUnit<BITS>;
    using SU = PairUnit<SW>;
    const NintDev& w = a.w;

    extern __shared__ __align__(16) unsigned char smem[];
    float* ypart = reinterpret_cast<float*>(smem);                       // [rb_per_cta][16]
    __nv_bfloat16* xs = reinterpret_cast<__nv_bfloat16*>(ypart + (size_t)a.rb_per_cta * 16);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarps = blockDim.x >> 5;
    const int q = lane >> 2, c = lane & 3;
    const int rb0 = blockIdx.x * a.rb_per_cta;
    const int nrb = min(a.rb_per_cta, w.nrb - rb0);

    const int my_segs = warp < w.nchunks ? (w.nchunks - warp + nwarps - 1) / nwarps : 0;
    const int n_mine = my_segs * nrb;
    auto item_seg = [&](int i) { return warp + (i / nrb) * nwarps; };
    auto item_rb = [&](int i) { return rb0 + i % nrb; };

    pdl_launch_dependents();
    Item it0, it1;
    if (0 < n_mine) it0.load(w, item_rb(0), item_seg(0), lane);
    if (1 < n_mine) it1.load(w, item_rb(1), item_seg(1), lane);
    for (int i = tid; i < nrb * 16; i += blockDim.x) ypart[i] = 0.f;
    pdl_wait();
    {   // stage x (zero beyond k): 16-byte copies when the row is 16-byte aligned
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
        float s[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int g = 0; g < 4; ++g) {
#pragma unroll
            for (int j = 0; j < HALF; ++j) {
                b0[g][j] = q == g ? xq[j] : 0u;
                b1[g][j] = q == g + 4 ? xq[j] : 0u;
                mma_k16(s, kBf16x2_one, kBf16x2_one, kBf16x2_one, kBf16x2_one, b0[g][j], b1[g][j]);
            }
        }
        xs0 = s[0];
        xs1 = s[1];
    };

    auto compute_item = [&](const Item& it, int rbl) {
        const float seed0 = (NPL == 2 ? -128.f * 17.f : -128.f) * xs0, seed1 = (NPL == 2 ? -128.f * 17.f : -128.f) * xs1;
        float acc_a[4] = {seed0, seed1, seed0, seed1}, acc_b[4] = {0.f, 0.f, 0.f, 0.f};
        float acc_c[4] = {0.f, 0.f, 0.f, 0.f}, acc_d[4] = {0.f, 0.f, 0.f, 0.f};   // high nibbles (8-bit codes)
#pragma unroll
        for (int g = 0; g < 4; ++g) {
#pragma unroll
            for (int j = 0; j < HALF; ++j) {
                const uint32_t r0 = QU::at(it.qw, (g * 2 + 0) * HALF + j), r1 = QU::at(it.qw, (g * 2 + 1) * HALF + j);
                const uint32_t r2 = QU::at(it.qw, ((g + 4) * 2 + 0) * HALF + j), r3 = QU::at(it.qw, ((g + 4) * 2 + 1) * HALF + j);
                if constexpr (NPL == 1) {
                    mma_k16(g < 2 ? acc_a : acc_b, r0 | kBf16x2_128, r1 | kBf16x2_128, r2 | kBf16x2_128, r3 | kBf16x2_128,
                            b0[g][j], b1[g][j]);
                } else {
                    constexpr uint32_t NIB = 0x000F000Fu;
                    mma_k16(g < 2 ? acc_a : acc_b, (r0 & NIB) | kBf16x2_128, (r1 & NIB) | kBf16x2_128, (r2 & NIB) | kBf16x2_128,
                            (r3 & NIB) | kBf16x2_128, b0[g][j], b1[g][j]);
                    mma_k16(g < 2 ? acc_c : acc_d, ((r0 >> 4) & NIB) | kBf16x2_128, ((r1 >> 4) & NIB) | kBf16x2_128,
                            ((r2 >> 4) & NIB) | kBf16x2_128, ((r3 >> 4) & NIB) | kBf16x2_128, b0[g][j], b1[g][j]);
                }
            }
        }
        float acc[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            acc[e] = acc_a[e] + acc_b[e];
            if constexpr (NPL == 2) acc[e] = fmaf(16.f, acc_c[e] + acc_d[e], acc[e]);
        }
        // sub-scales / sub-mins of rows (q, q+8) x groups (2c, 2c+1)
        uint32_t sp0, sp1, mp_lo, mp_hi;
        switch (c) {
            case 0: sp0 = SU::at(it.sw, 0); sp1 = SU::at(it.sw, 1); mp_lo = SU::at(it.sw, 8); mp_hi = SU::at(it.sw, 12); break;
            case 1: sp0 = SU::at(it.sw, 2); sp1 = SU::at(it.sw, 3); mp_lo = SU::at(it.sw, 9); mp_hi = SU::at(it.sw, 13); break;
            case 2: sp0 = SU::at(it.sw, 4); sp1 = SU::at(it.sw, 5); mp_lo = SU::at(it.sw, 10); mp_hi = SU::at(it.sw, 14); break;
            default: sp0 = SU::at(it.sw, 6); sp1 = SU::at(it.sw, 7); mp_lo = SU::at(it.sw, 11); mp_hi = SU::at(it.sw, 15); break;
        }
        float s0_lo, s0_hi, s1_lo, s1_hi, m0_lo, m1_lo, m0_hi, m1_hi;
        pair_to_floats<SW>(sp0, s0_lo, s0_hi);
        pair_to_floats<SW>(sp1, s1_lo, s1_hi);
        pair_to_floats<SW>(mp_lo, m0_lo, m1_lo);
        pair_to_floats<SW>(mp_hi, m0_hi, m1_hi);
        const __half2 h_lo = *reinterpret_cast<const __half2*>(&it.an_lo), h_hi = *reinterpret_cast<const __half2*>(&it.an_hi);
        const float2 f_lo = __half22float2(h_lo), f_hi = __half22float2(h_hi);  // (ns, nm)
        float v_lo = f_lo.x * fmaf(s1_lo, acc[1], s0_lo * acc[0]) - f_lo.y * fmaf(m1_lo, xs1, m0_lo * xs0);
        float v_hi = f_hi.x * fmaf(s1_hi, acc[3], s0_hi * acc[2]) - f_hi.y * fmaf(m1_hi, xs1, m0_hi * xs0);
        v_lo += __shfl_xor_sync(0xffffffffu, v_lo, 1);
        v_hi += __shfl_xor_sync(0xffffffffu, v_hi, 1);
        v_lo += __shfl_xor_sync(0xffffffffu, v_lo, 2);
        v_hi += __shfl_xor_sync(0xffffffffu, v_hi, 2);
        if (c == 0) {
            atomicAdd(ypart + rbl * 16 + q, v_lo);
            atomicAdd(ypart + rbl * 16 + q + 8, v_hi);
        }
    };

    for (int i = 0; i < n_mine; i += 2) {
        {
            const int seg = item_seg(i);
            if (seg != cur_seg) { cur_seg = seg; prepare_chunk(seg); }
            compute_item(it0, i % nrb);
            if (i + 2 < n_mine) it0.load(w, item_rb(i + 2), item_seg(i + 2), lane);
        }
        if (i + 1 < n_mine) {
            const int seg = item_seg(i + 1);
            if (seg != cur_seg) { cur_seg = seg; prepare_chunk(seg); }
            compute_item(it1, (i + 1) % nrb);
            if (i + 3 < n_mine) it1.load(w, item_rb(i + 3), item_seg(i + 3), lane);
        }
    }
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

}  // namespace mfqb
