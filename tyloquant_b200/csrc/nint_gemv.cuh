// Weight-streaming GEMV for NINT weights on mma.sync tensor-core tiles.
//
//   y[m, n] = sum_k x[m, k] * W[n, k],   W[n, k] = (ns[n]*ss[n,g]) * q[n,k] - (nm[n]*sm[n,g])
//
// is evaluated as   ns[n] * sum_g ss[n,g] * (sum_{k in g} q x)  -  nm[n] * sum_g sm[n,g] * xsum[g]
// with every inner sum in float32:
//   * the integer codes q go to the tensor cores as exact bf16 values (128 + q, built with one
//     logic op per code pair; the accumulator starts at -128 * xsum[g]), x as bf16, one
//     m16n8k16 / m16n8k8 chain per group of a 16-row block, batch rows (m <= 8) in the n8 slot;
//   * each group accumulator is scaled by its integer sub-scale on the CUDA cores;
//   * the sub-min term is a second small tensor-core product over the groups of a chunk, with
//     xsum split into three bf16 pieces (24 significant bits).
// A warp owns one chunk of 8 groups (its x fragments live in registers) and walks the CTA's
// row-blocks; partial sums of the chunks meet in shared memory.
// Replaces gemv_packed_* / gemv_packed_bits_* (mfq/kernels/cuda/nint_matmul.cu:1317-1383,
// 2598-2872) without their int8 activation quantization.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "common.h"
#include "nint_layout.h"
#include "pair_unit.h"

namespace mfqb {

__device__ __forceinline__ void mma_k16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                        uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void mma_k8(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t b0) {
    asm volatile(
        "mma.sync.aligned.m16n8k8.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%0,%1,%2,%3};\n"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(b0));
}

// First step of an accumulation chain: D = A*B + 0 (no accumulator registers to clear).
__device__ __forceinline__ void mma_k16_first(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                              uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};\n"
        : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.f));
}

constexpr uint32_t kBf16x2_128 = 0x43004300u;  // (128.0, 128.0)

__device__ __forceinline__ uint32_t bf162_sub128(uint32_t v) {
    __nv_bfloat162 a = *reinterpret_cast<__nv_bfloat162*>(&v);
    uint32_t c = kBf16x2_128;
    __nv_bfloat162 b = *reinterpret_cast<__nv_bfloat162*>(&c);
    __nv_bfloat162 r = __hsub2(a, b);
    return *reinterpret_cast<uint32_t*>(&r);
}

// Pair of small unsigned integers (low / high half) -> exact bf16x2.
template <int W>
__device__ __forceinline__ uint32_t pair_to_bf162(uint32_t raw) {
    if constexpr (W <= 7) {
        return bf162_sub128(raw | kBf16x2_128);
    } else {
        __nv_bfloat162 r = __floats2bfloat162_rn((float)(raw & 0xFFFFu), (float)(raw >> 16));
        return *reinterpret_cast<uint32_t*>(&r);
    }
}
template <int W>
__device__ __forceinline__ void pair_to_floats(uint32_t raw, float& lo, float& hi) {
    if constexpr (W <= 7) {
        const uint32_t u = bf162_sub128(raw | kBf16x2_128);
        lo = __uint_as_float(u << 16);
        hi = __uint_as_float(u & 0xFFFF0000u);
    } else {
        lo = (float)(raw & 0xFFFFu);
        hi = (float)(raw >> 16);
    }
}

__device__ __forceinline__ uint32_t pack_bf162(float lo, float hi) {
    __nv_bfloat162 r = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&r);
}

struct GemvArgs {
    NintDev w;
    const __nv_bfloat16* x;  // [m, k]
    void* y;                 // [m, ldy]
    int m, ldy, y_dtype;
    int rb_per_cta;          // row-blocks per CTA
    int xstride;             // row stride (elements, multiple of 8) of x staged in shared memory; 0 = read x from global
    int stages;              // records per warp ring (single-row kernel)
    // Routed mode of the single-row kernel (expert matmul, "mul_mat_id"): blockIdx.y is a
    // (token, route) pair; the pair's expert selects a block of rows_per_expert rows of w.
    // A CTA whose expert does not live in this cohort (pool) returns at once.
    const int* route_ids;    // [pairs] expert of each pair; nullptr = plain GEMV
    const int* expert_pool;  // [experts] cohort index of each expert (-1: not held here)
    const int* expert_local; // [experts] position of the expert inside its cohort
    int pool;                // cohort this launch covers
    int rb_per_expert;       // rows_per_expert / 16
    int routes;              // routes per token (R)
    int x_per_pair;          // 1: x is [pairs, k]; 0: x is [tokens, k], shared by the token's routes
    // Routed tile mode of the batched kernel: blockIdx.y is a tile of up to 8 pairs of one expert,
    // taken from a route plan (expert_bounds / tile_bounds / pair_order of mfqb_moe_route_plan).
    const int* expert_bounds;
    const int* tile_bounds;
    const int* pair_order;
    int n_experts;
};

constexpr uint32_t kBf16x2_one = 0x3F803F80u;  // (1.0, 1.0)

// Programmatic dependent launch: let the next kernel of the stream start early, and wait for
// the previous one before touching anything it may have produced.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

template <int BITS, int PER, int SW>
struct GemvItem {   // packed words of one (row-block, chunk) item, as loaded by one lane
    static constexpr int WC = PairUnit<BITS>::words_for(kChunkGroups * PER), SWC = PairUnit<SW>::words_for(16);
    uint32_t qw[WC], sw[SWC], an_lo, an_hi;
    __device__ __forceinline__ void load(const NintDev& w, int rb, int seg, int lane) {
        const uint32_t* rec = w.items + ((size_t)rb * w.nchunks + seg) * (WC * 32 + SWC * 8);
        const int q = lane >> 2;
#pragma unroll
        for (int j = 0; j < WC; ++j) qw[j] = __ldg(rec + j * 32 + lane);
#pragma unroll
        for (int j = 0; j < SWC; ++j) sw[j] = __ldg(rec + WC * 32 + j * 8 + q);
        an_lo = __ldg(w.anchors + rb * 16 + q);
        an_hi = __ldg(w.anchors + rb * 16 + 8 + q);
    }
};

// One CTA owns rb_per_cta row-blocks and all chunks of K.  Warp i takes chunks i, i + nwarps,
// ... and, for each, every row-block of the CTA (so its x fragments are built once per chunk).
// Each warp keeps two (chunk, row-block) items of packed words in flight in registers; the first
// two are requested before the kernel waits for its predecessor, since weights are constants.
// Shared memory: partial sums [rb_per_cta][16][8] float32, one 8x8 float32 tile per warp, and
// (when it fits) x staged as bf16 [m][xstride].
template <int BITS, int PER, int SW>
__global__ void __launch_bounds__(256, 2) nint_gemv_kernel(const GemvArgs a) {
    constexpr int G = kChunkGroups, HALF = PER / 2;
    constexpr int NPL = BITS == 8 ? 2 : 1;  // 8-bit codes go through as two 4-bit planes
    using Item = GemvItem<BITS, PER, SW>;
    using QU = PairUnit<BITS>;
    using SU = PairUnit<SW>;
    const NintDev& w = a.w;

    extern __shared__ __align__(16) unsigned char smem[];
    float* ypart = reinterpret_cast<float*>(smem);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarps = blockDim.x >> 5;
    const int q = lane >> 2, c = lane & 3;
    __shared__ int row_src[8], row_dst[8];   // x row read / y row written by batch column i
    int rb0 = blockIdx.x * a.rb_per_cta, rb_limit = w.nrb, m_cur = a.m, row_bias = 0, row_limit = w.n;
    if (a.tile_bounds != nullptr) {
        pdl_wait();   // the route plan comes from earlier kernels of the stream
        const int t = blockIdx.y;
        if (t >= a.tile_bounds[a.n_experts]) return;
        int lo = 0, hi = a.n_experts - 1;   // expert e with tile_bounds[e] <= t < tile_bounds[e + 1]
        while (lo < hi) {
            const int mid = (lo + hi + 1) >> 1;
            if (a.tile_bounds[mid] <= t) lo = mid; else hi = mid - 1;
        }
        const int e = lo;
        if (a.expert_pool[e] != a.pool) return;
        const int p0 = a.expert_bounds[e] + (t - a.tile_bounds[e]) * 8;
        m_cur = min(8, a.expert_bounds[e + 1] - p0);
        if (tid < 8) {
            const int pair = tid < m_cur ? a.pair_order[p0 + tid] : 0;
            row_src[tid] = a.x_per_pair ? pair : pair / a.routes;
            row_dst[tid] = pair;
        }
        const int base = a.expert_local[e] * a.rb_per_expert;
        rb0 = base + blockIdx.x * a.rb_per_cta;
        rb_limit = base + a.rb_per_expert;
        row_bias = base * 16;        // y rows are counted inside the expert
        row_limit = a.ldy;
    } else if (tid < 8) {
        row_src[tid] = tid;
        row_dst[tid] = tid;
    }
    const int nrb = min(a.rb_per_cta, rb_limit - rb0);
    if (nrb <= 0) return;
    float* xt = ypart + (size_t)a.rb_per_cta * 128 + warp * 64;
    __nv_bfloat16* xs = reinterpret_cast<__nv_bfloat16*>(ypart + (size_t)a.rb_per_cta * 128 + nwarps * 64);

    // items of this warp: i -> chunk warp + (i / nrb) * nwarps, row-block rb0 + i % nrb
    const int my_segs = warp < w.nchunks ? (w.nchunks - warp + nwarps - 1) / nwarps : 0;
    const int n_mine = my_segs * nrb;
    auto item_seg = [&](int i) { return warp + (i / nrb) * nwarps; };
    auto item_rb = [&](int i) { return rb0 + i % nrb; };

    pdl_launch_dependents();
    Item it0, it1;
    if (0 < n_mine) it0.load(w, item_rb(0), item_seg(0), lane);
    if (1 < n_mine) it1.load(w, item_rb(1), item_seg(1), lane);
    for (int i = tid; i < nrb * 128; i += blockDim.x) ypart[i] = 0.f;
    pdl_wait();
    __syncthreads();   // row_src / row_dst
    if (a.xstride > 0) {
        // stage x: 16-byte copies when rows are 16-byte aligned, zero beyond k
        const int kp = a.xstride;
        if ((w.k & 7) == 0 && (reinterpret_cast<uintptr_t>(a.x) & 15) == 0) {
            const int vec_per_row = kp / 8;
            for (int i = tid; i < m_cur * vec_per_row; i += blockDim.x) {
                const int m = i / vec_per_row, v = i % vec_per_row;
                uint4 val = make_uint4(0u, 0u, 0u, 0u);
                if (v * 8 < w.k) val = __ldg(reinterpret_cast<const uint4*>(a.x + (size_t)row_src[m] * w.k) + v);
                *reinterpret_cast<uint4*>(xs + (size_t)m * kp + v * 8) = val;
            }
        } else {
            for (int i = tid; i < m_cur * kp; i += blockDim.x) {
                const int m = i / kp, k = i % kp;
                xs[i] = k < w.k ? a.x[(size_t)row_src[m] * w.k + k] : __float2bfloat16(0.f);
            }
        }
    }
    __syncthreads();

    const bool has_col = q < m_cur;
    const bool even_k = (w.k & 1) == 0;
    const __nv_bfloat16* xcol = a.x + (size_t)row_src[q] * w.k;
    const uint32_t* xrow = reinterpret_cast<const uint32_t*>(xs + (size_t)q * a.xstride);
    int cur_seg = -1;
    uint32_t xf[G][HALF];
    float ci[G][2];
    uint32_t bmin[3];

    auto prepare_chunk = [&](int seg) {
        // x fragments of the chunk for batch column q
#pragma unroll
        for (int g = 0; g < G; ++g) {
            const int kbase = (seg * G + g) * w.gs + c * PER;
#pragma unroll
            for (int j = 0; j < HALF; ++j) {
                const int k0 = kbase + 2 * j;
                uint32_t v = 0u;
                if (has_col && (c * PER + 2 * j < w.gs)) {
                    if (a.xstride > 0) {
                        v = xrow[k0 >> 1];
                    } else if (k0 < w.k) {
                        if (even_k) {
                            v = __ldg(reinterpret_cast<const uint32_t*>(xcol + k0));
                        } else {
                            v = __ldg(reinterpret_cast<const unsigned short*>(xcol + k0));
                            if (k0 + 1 < w.k) v |= (uint32_t)__ldg(reinterpret_cast<const unsigned short*>(xcol + k0 + 1)) << 16;
                        }
                    }
                }
                xf[g][j] = v;
            }
        }
        // group sums of x through the tensor cores (A = ones): seeds of the accumulators
        __syncwarp();
#pragma unroll
        for (int g = 0; g < G; ++g) {
            float s[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int j = 0; j + 1 < HALF; j += 2)
                mma_k16(s, kBf16x2_one, kBf16x2_one, kBf16x2_one, kBf16x2_one, xf[g][j], xf[g][j + 1]);
            if constexpr (HALF & 1) mma_k8(s, kBf16x2_one, kBf16x2_one, xf[g][HALF - 1]);
            ci[g][0] = -128.f * s[0];
            ci[g][1] = -128.f * s[1];
            if (q == 0) *reinterpret_cast<float2*>(xt + g * 8 + 2 * c) = make_float2(s[0], s[1]);
        }
        __syncwarp();
        // sub-min operand: xsum of groups (2c, 2c+1) for column q, split in three bf16 pieces
        float v0 = xt[(2 * c) * 8 + q], v1 = xt[(2 * c + 1) * 8 + q];
#pragma unroll
        for (int s = 0; s < 3; ++s) {
            const __nv_bfloat16 h0 = __float2bfloat16_rn(v0), h1 = __float2bfloat16_rn(v1);
            v0 -= __bfloat162float(h0);
            v1 -= __bfloat162float(h1);
            __nv_bfloat162 pr;
            pr.x = h0;
            pr.y = h1;
            bmin[s] = *reinterpret_cast<uint32_t*>(&pr);
        }
    };

    auto compute_item = [&](const Item& it, int rbl) {
        float tot[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int g = 0; g < G; ++g) {
            float acc[NPL][4];
#pragma unroll
            for (int pl = 0; pl < NPL; ++pl) {
                acc[pl][0] = ci[g][0];
                acc[pl][1] = ci[g][1];
                acc[pl][2] = ci[g][0];
                acc[pl][3] = ci[g][1];
            }
#pragma unroll
            for (int j = 0; j + 1 < HALF; j += 2) {
                const uint32_t r0 = QU::at(it.qw, (g * 2 + 0) * HALF + j), r1 = QU::at(it.qw, (g * 2 + 1) * HALF + j);
                const uint32_t r2 = QU::at(it.qw, (g * 2 + 0) * HALF + j + 1), r3 = QU::at(it.qw, (g * 2 + 1) * HALF + j + 1);
                if constexpr (NPL == 1) {
                    mma_k16(acc[0], r0 | kBf16x2_128, r1 | kBf16x2_128, r2 | kBf16x2_128, r3 | kBf16x2_128, xf[g][j], xf[g][j + 1]);
                } else {
                    constexpr uint32_t NIB = 0x000F000Fu;
                    mma_k16(acc[0], (r0 & NIB) | kBf16x2_128, (r1 & NIB) | kBf16x2_128, (r2 & NIB) | kBf16x2_128,
                            (r3 & NIB) | kBf16x2_128, xf[g][j], xf[g][j + 1]);
                    mma_k16(acc[1], ((r0 >> 4) & NIB) | kBf16x2_128, ((r1 >> 4) & NIB) | kBf16x2_128,
                            ((r2 >> 4) & NIB) | kBf16x2_128, ((r3 >> 4) & NIB) | kBf16x2_128, xf[g][j], xf[g][j + 1]);
                }
            }
            if constexpr (HALF & 1) {
                constexpr int j = HALF - 1;
                const uint32_t r0 = QU::at(it.qw, (g * 2 + 0) * HALF + j), r1 = QU::at(it.qw, (g * 2 + 1) * HALF + j);
                if constexpr (NPL == 1) {
                    mma_k8(acc[0], r0 | kBf16x2_128, r1 | kBf16x2_128, xf[g][j]);
                } else {
                    constexpr uint32_t NIB = 0x000F000Fu;
                    mma_k8(acc[0], (r0 & NIB) | kBf16x2_128, (r1 & NIB) | kBf16x2_128, xf[g][j]);
                    mma_k8(acc[1], ((r0 >> 4) & NIB) | kBf16x2_128, ((r1 >> 4) & NIB) | kBf16x2_128, xf[g][j]);
                }
            }
            float s_lo, s_hi;
            pair_to_floats<SW>(SU::at(it.sw, g), s_lo, s_hi);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                float v = acc[0][e];
                if constexpr (NPL == 2) v = fmaf(16.f, acc[1][e], v);
                tot[e] = fmaf(e < 2 ? s_lo : s_hi, v, tot[e]);
            }
        }
        // sub-min term: rows (lo, hi) x groups (2c, 2c+1) of this chunk against xsum
        uint32_t m_lo, m_hi;
        switch (c) {
            case 0: m_lo = SU::at(it.sw, 8); m_hi = SU::at(it.sw, 12); break;
            case 1: m_lo = SU::at(it.sw, 9); m_hi = SU::at(it.sw, 13); break;
            case 2: m_lo = SU::at(it.sw, 10); m_hi = SU::at(it.sw, 14); break;
            default: m_lo = SU::at(it.sw, 11); m_hi = SU::at(it.sw, 15); break;
        }
        m_lo = pair_to_bf162<SW>(m_lo);
        m_hi = pair_to_bf162<SW>(m_hi);
        float mt[4] = {0.f, 0.f, 0.f, 0.f};
        mma_k8(mt, m_lo, m_hi, bmin[2]);
        mma_k8(mt, m_lo, m_hi, bmin[1]);
        mma_k8(mt, m_lo, m_hi, bmin[0]);

        const __half2 h_lo = *reinterpret_cast<const __half2*>(&it.an_lo), h_hi = *reinterpret_cast<const __half2*>(&it.an_hi);
        const float2 f_lo = __half22float2(h_lo), f_hi = __half22float2(h_hi);  // (ns, nm)
        float* yp = ypart + (size_t)rbl * 128;
        if (2 * c < m_cur) {
            atomicAdd(yp + q * 8 + 2 * c, f_lo.x * tot[0] - f_lo.y * mt[0]);
            atomicAdd(yp + (q + 8) * 8 + 2 * c, f_hi.x * tot[2] - f_hi.y * mt[2]);
        }
        if (2 * c + 1 < m_cur) {
            atomicAdd(yp + q * 8 + 2 * c + 1, f_lo.x * tot[1] - f_lo.y * mt[1]);
            atomicAdd(yp + (q + 8) * 8 + 2 * c + 1, f_hi.x * tot[3] - f_hi.y * mt[3]);
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
    const int rows = nrb * 16;
    for (int i = tid; i < rows * m_cur; i += blockDim.x) {
        const int n = i / rows, rr = i % rows, row = rb0 * 16 + rr - row_bias;
        if (row < row_limit) {
            const float v = ypart[rr * 8 + n];
            if (a.y_dtype == 0 /* MFQB_F32 */) reinterpret_cast<float*>(a.y)[(size_t)row_dst[n] * a.ldy + row] = v;
            else reinterpret_cast<__nv_bfloat16*>(a.y)[(size_t)row_dst[n] * a.ldy + row] = __float2bfloat16_rn(v);
        }
    }
}

// Shared-memory footprint and launch geometry, computed on the host.
struct GemvPlan {
    int rb_per_cta, grid, grid_y, threads, xstride, stages;
    size_t smem;
};
GemvPlan plan_nint_gemv(const NintDev& w, int m, int num_sms);

template <int BITS>
cudaError_t launch_nint_gemv_bits(const GemvArgs& a, const GemvPlan& p, cudaStream_t stream);

void launch_nint_gemv_routed(GemvArgs a, int pairs, int device, cudaStream_t s);
void launch_nint_gemv_routed_tiles(GemvArgs a, int max_tiles, int device, cudaStream_t s);
void launch_nint_dequant_view(const NintDev& w, void* out, int out_dtype, cudaStream_t s);
void check_nint_supported(const HostNint& t);

}  // namespace mfqb
