// Batched GEMV (2 to 8 activation rows per pass) for NINT weights in the byte-lane layout.
//
// Same integer pipeline as the single-row kernel (activation rows quantised per group to 16-bit
// integers, two byte planes, int8 tensor-core mma with a block-diagonal B), but the eight
// columns of a step (f, t) now carry two batch rows x the four groups of the family:
//
//   column n  ->  batch row 2p + (n >> 2),  group 4f + (n & 3)          (pass p = 0..P-1)
//
// so a pass of two rows costs as many mma as the single-row kernel and a batch of 2P rows
// decodes every weight once.  The accumulator fragment gives lane (q, c) the sums of weight
// rows q, q+8 for batch row 2p + (c>>1) and groups 4f + 2(c&1) + {0, 1}; the scale bytes of
// those (rows, groups) are the scale words of lane 4q + 2f + (c&1) of the record.  Lanes c and
// c^1 together hold the four groups of the family, so one shuffle finishes the sum over groups.
//
// The activation rows arrive already quantised (x_planes_kernel runs once per call, so a row
// shared by many CTAs is quantised once).  A warp owns whole chunks of K, as in the single-row
// kernel; together with the first weight record of a chunk it requests that chunk's planes of all
// batch rows ([row][group][quad] of (low, high) words plus the (scale, scaled sum) pairs, 64*(QS+1)
// bytes per row) into one of its two private plane buffers with the same asynchronous copies, so
// no CTA-wide barrier separates the warps while they stream.
//
// Tile mode (expert matmul with a route plan): blockIdx.y is a tile of up to 2P (token, route)
// pairs of one expert; x rows are gathered through pair_order and results scatter back to pair
// order.  The route plan's tile size must equal 2P.
#pragma once
#include "nint_gemv1_bl.cuh"

namespace mfqb {

// Quantises rows of x into the global plane buffers the batched kernel reads: grid = (K splits,
// rows), every CTA a range of whole chunks.
template <int T, typename XT>
__global__ void __launch_bounds__(256) x_planes_kernel(const XT* __restrict__ x, int k, int gs, int ngp, int groups_per_cta,
                                                       uint2* __restrict__ xq_g, float2* __restrict__ gtab_g) {
    constexpr int QS = gemv1_bl_qstride(T);
    const int row = blockIdx.y, g0 = blockIdx.x * groups_per_cta;
    if (g0 >= ngp) return;
    stage_x_planes<T, XT>(x + (size_t)row * k, k, gs, g0, min(groups_per_cta, ngp - g0), xq_g + ((size_t)row * ngp + g0) * QS,
                          gtab_g + (size_t)row * ngp + g0);
}

// Ring depth of the batched kernel (the plane buffers take the shared memory of one or two stages).
__host__ __device__ constexpr int gemvn_bl_stages(int rec_words, int passes) {
    return gemv1_bl_stages(rec_words) > (passes >= 4 ? 3 : 4) ? (passes >= 4 ? 3 : 4) : gemv1_bl_stages(rec_words);
}
// Bytes of one batch row of one chunk in a plane buffer: 8 groups x QS quads of (low, high) words, then 8 (scale, scaled sum) pairs.
__host__ __device__ constexpr int gemvn_bl_row_bytes(int t8) { return 64 * (gemv1_bl_qstride(t8) + 1); }

template <class C, int P>
__device__ __forceinline__ void gemvn_bl_body(const GemvArgsB& a, const NintDevB& w, unsigned char* smem) {
    constexpr int G = kChunkGroupsB, MB = 2 * P, T = C::T, WC = C::WC, SW = C::SW, REC = (WC + SW) * 32;
    constexpr int S = gemvn_bl_stages(REC, P), QS = gemv1_bl_qstride(T), PLB = gemvn_bl_row_bytes(T);

    __shared__ int row_src[MB], row_dst[MB];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarps = blockDim.x >> 5;
    const int q = lane >> 2, c = lane & 3;
    const int ystride = a.rb_per_cta * 16;
    typename C::Ctx ctx;
    ctx.init(smem, w, tid, blockDim.x);   // constant tables: visible after the first __syncthreads
    float* ypart = reinterpret_cast<float*>(smem + C::ctx_bytes(w));                // [MB][rb_per_cta * 16]
    uint32_t* anch = reinterpret_cast<uint32_t*>(ypart + (size_t)MB * ystride);     // [rb_per_cta * 16]
    unsigned char* planes_all = reinterpret_cast<unsigned char*>(anch + ystride);   // [warp][2 buffers][MB rows][PLB]
    unsigned char* planes = planes_all + (size_t)warp * 2 * MB * PLB;
    uint32_t* ring = reinterpret_cast<uint32_t*>(planes_all + (size_t)nwarps * 2 * MB * PLB) + (size_t)warp * S * REC;

    int m_cur = a.m, rb0, nrb, rbl0 = 0, row_limit = w.n;
    pdl_wait_b();   // the quantised planes (and, in tile mode, the route plan) come from the previous kernels
    if (a.tile_bounds != nullptr) {
        const int t = blockIdx.y;
        if (t >= a.tile_bounds[a.n_experts]) return;
        int lo = 0, hi = a.n_experts - 1;   // expert e with tile_bounds[e] <= t < tile_bounds[e + 1]
        while (lo < hi) {
            const int mid = (lo + hi + 1) >> 1;
            if (a.tile_bounds[mid] <= t) lo = mid;
            else hi = mid - 1;
        }
        const int e = lo;
        if (a.expert_pool[e] != a.pool) return;
        const int p0 = a.expert_bounds[e] + (t - a.tile_bounds[e]) * MB;
        m_cur = min(MB, a.expert_bounds[e + 1] - p0);
        if (tid < MB) {
            const int pair = tid < m_cur ? a.pair_order[p0 + tid] : 0;
            row_src[tid] = a.x_per_pair ? pair : pair / a.routes;
            row_dst[tid] = pair;
        }
        split_row_blocks(blockIdx.x, gridDim.x, a.rb_per_expert, rbl0, nrb);
        rb0 = a.expert_local[e] * a.rb_per_expert + rbl0;
        row_limit = a.ldy;
    } else {
        if (tid < MB) row_src[tid] = row_dst[tid] = tid;
        split_row_blocks(blockIdx.x, gridDim.x, w.nrb, rbl0, nrb);
        rb0 = rbl0;
    }
    pdl_launch_dependents_b();
    for (int i = tid; i < MB * ystride; i += blockDim.x) ypart[i] = 0.f;
    for (int i = tid; i < nrb * 16; i += blockDim.x) anch[i] = __ldg(w.anchors + rb0 * 16 + i);
    // rows past the batch are never copied: their planes and scale pairs stay zero and contribute nothing
    for (int i = tid; i < nwarps * 2 * MB * PLB / 16; i += blockDim.x) reinterpret_cast<uint4*>(planes_all)[i] = make_uint4(0u, 0u, 0u, 0u);
    __syncthreads();   // row_src / row_dst, zeroed buffers

    // items of this warp, chunk-major: chunk = warp, warp + nwarps, ...; inside a chunk every
    // row-block of the CTA.  The issue cursor runs `ahead` <= min(S, nrb) items in front, so the
    // items in flight touch at most two chunks: the two plane buffers alternate by chunk.
    const int my_segs = warp < w.nchunks ? (w.nchunks - warp + nwarps - 1) / nwarps : 0;
    const int n_mine = my_segs * nrb, ahead = min(S, nrb), ngp = w.nchunks * G;
    int iss_i = 0, iss_seg = warp, iss_rbl = 0, iss_stage = 0, iss_buf = 0;
    auto issue = [&]() {
        if (iss_i < n_mine) {
            const uint32_t* src = w.items + ((size_t)(rb0 + iss_rbl) * w.nchunks + iss_seg) * REC;
            uint32_t* dst = ring + iss_stage * REC;
#pragma unroll
            for (int off = 0; off < REC; off += 128)
                if (off + 128 <= REC || lane * 4 < REC - off) cp_async16_b(dst + off + lane * 4, src + off + lane * 4);
            if (iss_rbl == 0) {   // first item of a chunk: its planes travel in the same group
                unsigned char* pb = planes + (size_t)iss_buf * MB * PLB;
                constexpr int PIECES = 4 * QS + 4;   // 16-byte pieces per batch row
                for (int idx = lane; idx < m_cur * PIECES; idx += 32) {
                    const int m = idx / PIECES, piece = idx % PIECES;
                    const size_t grp0 = (size_t)row_src[m] * ngp + (size_t)iss_seg * G;
                    const unsigned char* gsrc = piece < 4 * QS ? reinterpret_cast<const unsigned char*>(a.xq_g + grp0 * QS) + piece * 16
                                                               : reinterpret_cast<const unsigned char*>(a.gtab_g + grp0) + (piece - 4 * QS) * 16;
                    cp_async16_b(pb + m * PLB + piece * 16, gsrc);
                }
                iss_buf ^= 1;
            }
        }
        cp_async_commit_b();   // one group per item slot, empty past the end: keeps the wait count uniform
        ++iss_i;
        if (++iss_rbl == nrb) { iss_rbl = 0; iss_seg += nwarps; }
        if (++iss_stage == S) iss_stage = 0;
    };
    for (int i = 0; i < ahead; ++i) issue();

    // B masks: lane (q, c) feeds column q = (batch row q>>2 of the pass, octet o = q&3); its bytes
    // are live in b0 where the fragment's octet c>>1 is o (o < 2), in b1 where 2 + (c>>1) is o
    const int o = q & 3;
    const bool live = (o & 1) == (c >> 1);
    const uint32_t mA = (live && o < 2) ? 0xFFFFFFFFu : 0u, mB = (live && o >= 2) ? 0xFFFFFFFFu : 0u;

    int rbl = 0, stage = 0, buf = 0;
    for (int i = 0; i < n_mine; ++i) {
        // the groups newer than this item's are the ahead - 1 items issued after it
        switch (ahead) {
            case 1: asm volatile("cp.async.wait_group 0;\n" ::: "memory"); break;
            case 2: asm volatile("cp.async.wait_group 1;\n" ::: "memory"); break;
            case 3: asm volatile("cp.async.wait_group 2;\n" ::: "memory"); break;
            default: asm volatile("cp.async.wait_group 3;\n" ::: "memory"); break;
        }
        __syncwarp();
        const uint32_t* rec = ring + stage * REC;
        const unsigned char* pb = planes + (size_t)buf * MB * PLB;
        uint32_t qw[WC];
#pragma unroll
        for (int j = 0; j < WC; ++j) qw[j] = rec[j * 32 + lane];
        uint32_t sc[2][SW], own[SW];   // scale words of the lanes that own (rows q, q+8) x groups 4f + 2(c&1) + {0,1}; this lane's
#pragma unroll
        for (int f = 0; f < 2; ++f)
#pragma unroll
            for (int j = 0; j < SW; ++j) sc[f][j] = rec[(WC + j) * 32 + 4 * q + 2 * f + (c & 1)];
#pragma unroll
        for (int j = 0; j < SW; ++j) own[j] = C::NEEDS_OWN_SCALE ? rec[(WC + j) * 32 + lane] : 0u;
        __syncwarp();          // every lane has read the stage before it is refilled
        issue();               // item i + ahead: never into the plane buffer this item reads (see above)

        float A_lo[P], A_hi[P], M_lo[P], M_hi[P];
#pragma unroll
        for (int p = 0; p < P; ++p) A_lo[p] = A_hi[p] = M_lo[p] = M_hi[p] = 0.f;
#pragma unroll
        for (int f = 0; f < 2; ++f) {
            int dlo[P][4], dhi[P][4];
#pragma unroll
            for (int p = 0; p < P; ++p)
#pragma unroll
                for (int e = 0; e < 4; ++e) dlo[p][e] = dhi[p][e] = 0;
#pragma unroll
            for (int t = 0; t < T; ++t) {
                const int r = (f * T + t) * 4;
                const uint32_t a0 = C::areg(qw, r, ctx, own), a1 = C::areg(qw, r + 1, ctx, own), a2 = C::areg(qw, r + 2, ctx, own),
                               a3 = C::areg(qw, r + 3, ctx, own);
#pragma unroll
                for (int p = 0; p < P; ++p) {
                    const uint2 v = *reinterpret_cast<const uint2*>(pb + (2 * p + (q >> 2)) * PLB + ((4 * f + o) * QS + 2 * t + (c & 1)) * 8);
                    imma_planes<C::A_SIGNED>(dlo[p], dhi[p], a0, a1, a2, a3, v.x & mA, v.x & mB, v.y & mA, v.y & mB);
                }
            }
            float ss[4], sm[4];
            C::scales(sc[f], ctx, ss, sm);
#pragma unroll
            for (int p = 0; p < P; ++p) {
                // (sx, sx*X) of groups 4f + 2(c&1) + {0,1} for batch row 2p + (c>>1)
                const float4 gt = *reinterpret_cast<const float4*>(pb + (2 * p + (c >> 1)) * PLB + 64 * QS + (4 * f + 2 * (c & 1)) * 8);
                const float d0 = (float)(dhi[p][0] * 256 + dlo[p][0]) * gt.x, d1 = (float)(dhi[p][1] * 256 + dlo[p][1]) * gt.z;
                const float d2 = (float)(dhi[p][2] * 256 + dlo[p][2]) * gt.x, d3 = (float)(dhi[p][3] * 256 + dlo[p][3]) * gt.z;
                A_lo[p] = fmaf(ss[1], d1, fmaf(ss[0], d0, A_lo[p]));
                A_hi[p] = fmaf(ss[3], d3, fmaf(ss[2], d2, A_hi[p]));
                if constexpr (C::HAS_MIN) {
                    M_lo[p] = fmaf(sm[1], gt.w, fmaf(sm[0], gt.y, M_lo[p]));
                    M_hi[p] = fmaf(sm[3], gt.w, fmaf(sm[2], gt.y, M_hi[p]));
                }
            }
        }
        const uint32_t an_lo = anch[rbl * 16 + q], an_hi = anch[rbl * 16 + q + 8];
        const float2 f_lo = __half22float2(*reinterpret_cast<const __half2*>(&an_lo));   // (ns, nm)
        const float2 f_hi = __half22float2(*reinterpret_cast<const __half2*>(&an_hi));
#pragma unroll
        for (int p = 0; p < P; ++p) {
            float v_lo = f_lo.x * A_lo[p] - f_lo.y * M_lo[p];
            float v_hi = f_hi.x * A_hi[p] - f_hi.y * M_hi[p];
            v_lo += __shfl_xor_sync(0xffffffffu, v_lo, 1);   // lanes c, c^1: the other two groups of each family
            v_hi += __shfl_xor_sync(0xffffffffu, v_hi, 1);
            const int m = 2 * p + (c >> 1);
            if ((c & 1) == 0 && m < m_cur) {
                atomicAdd(ypart + (size_t)m * ystride + rbl * 16 + q, v_lo);
                atomicAdd(ypart + (size_t)m * ystride + rbl * 16 + q + 8, v_hi);
            }
        }
        if (++rbl == nrb) { rbl = 0; buf ^= 1; }
        if (++stage == S) stage = 0;
    }
    asm volatile("cp.async.wait_group 0;\n" ::: "memory");
    __syncthreads();
    for (int i = tid; i < m_cur * nrb * 16; i += blockDim.x) {
        const int m = i / (nrb * 16), j = i % (nrb * 16);
        const int row = rbl0 * 16 + j;   // row inside the problem (matrix, or the tile's expert)
        if (row < row_limit) {
            const float v = ypart[(size_t)m * ystride + j] * kXScaleUndo;
            const size_t off = (size_t)row_dst[m] * a.ldy + row;
            if (a.y_dtype == 0 /* MFQB_F32 */) reinterpret_cast<float*>(a.y)[off] = v;
            else reinterpret_cast<__nv_bfloat16*>(a.y)[off] = __float2bfloat16_rn(v);
        }
    }
}

template <class C, int P>
__global__ void __launch_bounds__(256, (P >= 4 || C::MIN_CTAS < 3) ? (C::MIN_CTAS < 2 ? 1 : 2) : 3) gemvn_bl_kernel(const GemvArgsB a) {
    extern __shared__ __align__(16) unsigned char smem[];
    gemvn_bl_body<C, P>(a, a.w, smem);
}

}  // namespace mfqb
