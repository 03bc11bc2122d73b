// Batched GEMV (5 to 16 activation rows per launch) with the weights dequantised to f16 in registers.
//
// The integer kernels put the eight groups of a chunk (single row) or two batch rows x four groups
// (batched) into the n8 slot of the int8 mma, because group scales have to be applied to integer
// sums.  From eight batch rows on it pays to apply the scales to the weights instead: a lane turns
// each of its byte-lane registers (four codes of one weight row and group) into two f16x2
// registers w = d * q - m, which ARE the A fragment of mma.m16n8k16 (f16 x f16 -> f32), and the
// eight columns carry eight batch rows.  One byte-lane step (f, t) -- rows q, q+8 x groups
// 4f + (c>>1), 4f + 2 + (c>>1) x slots 8t + 4(c&1) + {0..3} -- is two such mma per eight batch
// rows (codes 0,1 are the fragment's k = 2c, 2c+1, codes 2,3 its k = 2c+8, 2c+9; the k order of
// an mma is free as long as B follows it), 4T mma per record instead of 4T per two rows, and the
// accumulators are final values: no per-group scaling afterwards.
//
// Activations: every row is scaled by a power of two so that its largest magnitude lands near 2^14
// (x_row_scale_kernel; the inverse factor is applied to the finished sums) and written as f16 in the
// order the B fragments are consumed (x_frag_kernel): per tile of 8 NT rows and chunk, for each mma
// of the record the 32 lanes' 8 bytes next to each other, so a warp fetches a fragment with one
// coalesced 256-byte read that the other row-blocks of the chunk and the other CTAs of the tile find
// in L1 / L2 -- no shared-memory staging, which leaves room for four CTAs per SM.  Exact for a bf16
// input within 2^-28 of the row's largest magnitude.  Weights are rounded to f16 once (d and the
// centred offset rounded to f16, one fused multiply-add): about 3e-4 relative L2 on the product,
// inside the path's 1e-3 bound.
//
// Tile mode (expert matmul with a route plan): blockIdx.y is a tile of up to 8 NT (token, route)
// pairs of one expert; x rows are taken through pair_order and results scatter back to pair order.
#pragma once
#include <cuda_fp16.h>

#include "nint_gemv1_bl.cuh"

namespace mfqb {

__host__ __device__ constexpr int gemvh_stages(int rec_words) { return gemv1_bl_stages(rec_words) > 4 ? 4 : gemv1_bl_stages(rec_words); }

// The dequantised weights carry a factor 2^10 (taken out of the finished sums): f16 then keeps all its
// bits for quantisation steps down to 2^-24 and represents weights up to 64.
constexpr float kGemvhWeightScale = 1024.f, kGemvhWeightUndo = 1.f / 1024.f;

__device__ __forceinline__ void hmma_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Four codes of a byte-lane register -> two f16x2 registers of d * (q - QMID) + nm, codes (0,1) and (2,3).
// A byte b becomes the f16 1024 + b by placing it under the exponent byte 0x64 (signed codes are
// biased by 128 first); subtracting 1024 + QMID is exact.  Centring the codes keeps d * (q - QMID)
// and nm = -(m - d * QMID) of the size of the weight itself, so the f16 roundings are relative to
// the weight and not to the (larger) offset of an asymmetric code range.
template <bool SIGNED, bool HAS_MIN, int QMID>
__device__ __forceinline__ void codes_to_f16(uint32_t v, __half2 d, __half2 nm, uint32_t& w01, uint32_t& w23) {
    if (SIGNED) v ^= 0x80808080u;
    const uint32_t lo = __byte_perm(v, 0x64646464u, 0x4140), hi = __byte_perm(v, 0x64646464u, 0x4342);
    const __half2 bias = __float2half2_rn((SIGNED ? 1152.f : 1024.f) + (float)QMID);
    const __half2 q01 = __hsub2(*reinterpret_cast<const __half2*>(&lo), bias), q23 = __hsub2(*reinterpret_cast<const __half2*>(&hi), bias);
    const __half2 r01 = HAS_MIN ? __hfma2(q01, d, nm) : __hmul2(q01, d), r23 = HAS_MIN ? __hfma2(q23, d, nm) : __hmul2(q23, d);
    w01 = *reinterpret_cast<const uint32_t*>(&r01);
    w23 = *reinterpret_cast<const uint32_t*>(&r23);
}

// Shared memory: partial sums [8 NT][rb_per_cta * 16] f32 | anchors [rb_per_cta * 16] | per warp a ring of S records.
template <class C, int NT>
__device__ __forceinline__ void gemvh_bl_body(const GemvArgsB& a, const NintDevB& w, unsigned char* smem) {
    constexpr int G = kChunkGroupsB, MB = 8 * NT, T = C::T, WC = C::WC, SW = C::SW, REC = (WC + SW) * 32;
    constexpr int S = gemvh_stages(REC), FRAGS = 4 * T * NT * 32;   // 8-byte units of one chunk of a tile

    __shared__ int row_src[MB], row_dst[MB];
    __shared__ float row_undo[MB];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarps = blockDim.x >> 5;
    const int q = lane >> 2, c = lane & 3;
    const int ystride = a.rb_per_cta * 16;
    typename C::Ctx ctx;
    ctx.init(smem, w, tid, blockDim.x);   // constant tables: visible after the first __syncthreads
    float* ypart = reinterpret_cast<float*>(smem + C::ctx_bytes(w));                // [MB][rb_per_cta * 16]
    uint32_t* anch = reinterpret_cast<uint32_t*>(ypart + (size_t)MB * ystride);     // [rb_per_cta * 16]
    uint32_t* ring = anch + ystride + (size_t)warp * S * REC;

    int m_cur = a.m, rb0, nrb, rbl0 = 0, row_limit = w.n;
    const uint2* xf = a.x16f;   // this tile's fragments
    pdl_wait_b();   // the fragments (and, in tile mode, the route plan) come from the previous kernels
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
        xf += (size_t)t * a.x16f_tile_stride;
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
    __syncthreads();   // row_src / row_dst
    if (tid < MB) row_undo[tid] = tid < m_cur ? a.x16_scale[row_src[tid]] * kGemvhWeightUndo : 0.f;

    // items of this warp, chunk-major: chunk = warp, warp + nwarps, ...; inside a chunk every
    // row-block of the CTA.  The issue cursor runs `ahead` = S items in front.
    const int my_segs = warp < w.nchunks ? (w.nchunks - warp + nwarps - 1) / nwarps : 0;
    const int n_mine = my_segs * nrb, ahead = S;
    int iss_i = 0, iss_seg = warp, iss_rbl = 0, iss_stage = 0;
    auto issue = [&]() {
        if (iss_i < n_mine) {
            const uint32_t* src = w.items + ((size_t)(rb0 + iss_rbl) * w.nchunks + iss_seg) * REC;
            uint32_t* dst = ring + iss_stage * REC;
#pragma unroll
            for (int off = 0; off < REC; off += 128)
                if (off + 128 <= REC || lane * 4 < REC - off) cp_async16_b(dst + off + lane * 4, src + off + lane * 4);
        }
        cp_async_commit_b();   // one group per item slot, empty past the end: keeps the wait count uniform
        ++iss_i;
        if (++iss_rbl == nrb) { iss_rbl = 0; iss_seg += nwarps; }
        if (++iss_stage == S) iss_stage = 0;
    };
    for (int i = 0; i < ahead; ++i) issue();

    int rbl = 0, stage = 0, seg = warp;
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
        const uint2* xc = xf + (size_t)seg * FRAGS + lane;   // the chunk's fragments, this lane's 8 bytes of each
        uint32_t qw[WC];
#pragma unroll
        for (int j = 0; j < WC; ++j) qw[j] = rec[j * 32 + lane];
        // scale words of the lanes that own (rows q, q+8) x groups 4f + 2h + {0, 1}; this lane's own
        uint32_t sc[2][2][SW], own[SW];
#pragma unroll
        for (int f = 0; f < 2; ++f)
#pragma unroll
            for (int h = 0; h < 2; ++h)
#pragma unroll
                for (int j = 0; j < SW; ++j) sc[f][h][j] = rec[(WC + j) * 32 + 4 * q + 2 * f + h];
#pragma unroll
        for (int j = 0; j < SW; ++j) own[j] = C::NEEDS_OWN_SCALE ? rec[(WC + j) * 32 + lane] : 0u;
        __syncwarp();          // every lane has read the stage before it is refilled
        issue();               // item i + ahead

        const uint32_t an_lo = anch[rbl * 16 + q], an_hi = anch[rbl * 16 + q + 8];
        const float2 f_lo = __half22float2(*reinterpret_cast<const __half2*>(&an_lo));   // (ns, nm)
        const float2 f_hi = __half22float2(*reinterpret_cast<const __half2*>(&an_hi));
        float acc[NT][4];
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.f;
        const bool odd = (c >> 1) != 0;   // this lane's group of a pair: 4f + 2h + (c>>1)
#pragma unroll
        for (int f = 0; f < 2; ++f) {
            // (d, -m) of rows q and q+8 for the two groups this lane decodes in family f
            __half2 d_lo[2], d_hi[2], nm_lo[2], nm_hi[2];
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                float s_lo, s_hi, m_lo = 0.f, m_hi = 0.f;   // sub-scale and sub-min of rows q, q+8 for this lane's group
                if constexpr (!C::A_SIGNED && C::SW == 2) {
                    // scalar codes: word 0 holds the four sub-scale bytes (row q even, odd group; row q+8 even, odd), word 1 the sub-mins
                    const uint32_t sh = odd ? 8u : 0u;
                    s_lo = (float)((sc[f][h][0] >> sh) & 0xFFu);
                    s_hi = (float)((sc[f][h][0] >> (sh + 16u)) & 0xFFu);
                    m_lo = (float)((sc[f][h][1] >> sh) & 0xFFu);
                    m_hi = (float)((sc[f][h][1] >> (sh + 16u)) & 0xFFu);
                } else {
                    float ss[4], sm[4];
                    C::scales(sc[f][h], ctx, ss, sm);
                    s_lo = odd ? ss[1] : ss[0];
                    s_hi = odd ? ss[3] : ss[2];
                    if constexpr (C::HAS_MIN) {
                        m_lo = odd ? sm[1] : sm[0];
                        m_hi = odd ? sm[3] : sm[2];
                    }
                }
                const float dl = kGemvhWeightScale * f_lo.x * s_lo, dh = kGemvhWeightScale * f_hi.x * s_hi;
                d_lo[h] = __float2half2_rn(dl);
                d_hi[h] = __float2half2_rn(dh);
                if constexpr (C::HAS_MIN) {
                    nm_lo[h] = __float2half2_rn(fmaf(dl, (float)C::QMID, -kGemvhWeightScale * f_lo.y * m_lo));
                    nm_hi[h] = __float2half2_rn(fmaf(dh, (float)C::QMID, -kGemvhWeightScale * f_hi.y * m_hi));
                } else {
                    nm_lo[h] = nm_hi[h] = __float2half2_rn(0.f);
                }
            }
#pragma unroll
            for (int t = 0; t < T; ++t) {
                const int r = (f * T + t) * 4;
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    // registers r + 2h (row q) and r + 2h + 1 (row q + 8): group 4f + 2h + (c>>1), slots 8t + 4(c&1) + {0..3}
                    uint32_t a0, a1, a2, a3;
                    codes_to_f16<C::A_SIGNED, C::HAS_MIN, C::QMID>(C::areg(qw, r + 2 * h, ctx, own), d_lo[h], nm_lo[h], a0, a2);
                    codes_to_f16<C::A_SIGNED, C::HAS_MIN, C::QMID>(C::areg(qw, r + 2 * h + 1, ctx, own), d_hi[h], nm_hi[h], a1, a3);
#pragma unroll
                    for (int nt = 0; nt < NT; ++nt) {
                        const uint2 b = __ldg(xc + (((f * T + t) * 2 + h) * NT + nt) * 32);
                        hmma_16816(acc[nt], a0, a1, a2, a3, b.x, b.y);
                    }
                }
            }
        }
        // acc[nt]: rows q (0, 1) and q+8 (2, 3) x batch rows 8 nt + 2c + {0, 1}
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            const int m0 = 8 * nt + 2 * c;
            if (m0 < m_cur) {
                atomicAdd(ypart + (size_t)m0 * ystride + rbl * 16 + q, acc[nt][0]);
                atomicAdd(ypart + (size_t)m0 * ystride + rbl * 16 + q + 8, acc[nt][2]);
            }
            if (m0 + 1 < m_cur) {
                atomicAdd(ypart + (size_t)(m0 + 1) * ystride + rbl * 16 + q, acc[nt][1]);
                atomicAdd(ypart + (size_t)(m0 + 1) * ystride + rbl * 16 + q + 8, acc[nt][3]);
            }
        }
        if (++rbl == nrb) { rbl = 0; seg += nwarps; }
        if (++stage == S) stage = 0;
    }
    asm volatile("cp.async.wait_group 0;\n" ::: "memory");
    __syncthreads();
    for (int i = tid; i < m_cur * nrb * 16; i += blockDim.x) {
        const int m = i / (nrb * 16), j = i % (nrb * 16);
        const int row = rbl0 * 16 + j;   // row inside the problem (matrix, or the tile's expert)
        if (row < row_limit) {
            const float v = ypart[(size_t)m * ystride + j] * row_undo[m];
            const size_t off = (size_t)row_dst[m] * a.ldy + row;
            if (a.y_dtype == 0 /* MFQB_F32 */) reinterpret_cast<float*>(a.y)[off] = v;
            else reinterpret_cast<__nv_bfloat16*>(a.y)[off] = __float2bfloat16_rn(v);
        }
    }
}

template <class C, int NT>
__global__ void __launch_bounds__(256, C::MIN_CTAS < 2 ? 1 : (NT == 1 ? 3 : 2)) gemvh_bl_kernel(const GemvArgsB a) {
    extern __shared__ __align__(16) unsigned char smem[];
    gemvh_bl_body<C, NT>(a, a.w, smem);
}

}  // namespace mfqb
