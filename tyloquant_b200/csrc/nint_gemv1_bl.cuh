// Single-row (m = 1) GEMV for weights in the byte-lane layout (NINT codes, or lattice vectors
// through a codec): the decode hot path.
//
// The weights never leave the integer domain.  The activation row is quantised, by the warp
// that needs it, group by group, to 16-bit integers  x_k ~ sx_g * xi_k  (sx_g a power of two chosen from the
// group's largest magnitude, so a bf16 input is reproduced exactly unless it is more than 2^7
// below that magnitude) and split into a low unsigned and a high signed byte plane.  The int8
// tensor-core instruction mma.m16n8k32 then forms  D[row][g] = sum_k q[row][k] * xi[k]  exactly:
// with one activation row the n8 slot of the tile is free, so the eight columns carry the eight
// *groups* of a chunk.  The B operand is block-diagonal (column g holds x only at the k-slots of
// group g), and one accumulator tile per byte plane collects all groups of the chunk.  The
// per-group integer sub-scales and sub-mins and the row anchors are applied once per chunk in
// float32 -- lane (q, c) owns groups 2c, 2c+1 of rows q, q+8, exactly the scale bytes its two
// private scale words hold -- and a quad reduction adds the eight groups:
//
//   y[row] = sum_g sx_g * ( ns*ss_g * D[row][g]  -  nm*sm_g * X_g ),     X_g = sum_k xi_k.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "comm_dev.cuh"
#include "common.h"
#include "lane_unit.h"
#include "nint_blayout.h"

namespace mfqb {

// Writes the scaled f16 activations in fragment order.  Grid (chunks, tiles), 256 threads.  A tile is
// 8 nt rows: the whole batch of a plain product (tile_bounds == nullptr, rows 0 .. m-1), or a route-plan
// tile of one expert, whose cohort fixes the geometry (octets per group T, chunks per row).  Layout of a
// tile, in 8-byte units: [chunk][mma j = (f T + t) 2 + h][row octet][lane], lane (q, c) holding row 8 nt + q,
// elements (4f + 2h + (c>>1)) 8T + 8t + 4(c&1) + {0..3} of the chunk.
struct XFragArgs {
    const void* x;        // [in_rows][k] bf16 or float32
    int x_f32, k;
    const float* up;      // scale of every source row
    uint2* out;
    size_t tile_stride;   // 8-byte units
    int nt, m;
    const int *expert_bounds, *tile_bounds, *pair_order, *expert_pool;
    int n_experts, routes, x_per_pair;
    int pool_t8[16], pool_nchunks[16];   // by cohort; a plain product uses entry 0
};
// One weight of a multi-weight launch (several weights of one shape class applied to the same x).
struct GemvMultiEntry {
    const uint32_t* items;
    const uint32_t* anchors;
    void* y;
    int n, nrb;
};
constexpr int kGemvMultiMax = 8;
struct GemvMultiTable {
    GemvMultiEntry e[kGemvMultiMax];
};

struct GemvArgsB {
    NintDevB w;
    const __nv_bfloat16* x;  // [m, k]
    void* y;                 // [m, ldy]
    int m, ldy, y_dtype;
    int rb_per_cta;          // row-blocks per CTA (upper bound; the kernel splits evenly)
    // Routed mode (expert matmul, "mul_mat_id"): blockIdx.y is a (token, route) pair; the pair's
    // expert selects a block of rb_per_expert row-blocks of w.  A CTA whose expert does not
    // live in this cohort (pool) returns at once.
    const int* route_ids;    // [pairs] expert of each pair; nullptr = plain GEMV
    const int* expert_pool;  // [experts] cohort index of each expert (-1: not held here)
    const int* expert_local; // [experts] position of the expert inside its cohort
    int pool;                // cohort this launch covers
    int rb_per_expert;       // rows_per_expert / 16
    int routes;              // routes per token (R)
    int x_per_pair;          // 1: x is [pairs, k]; 0: x is [tokens, k], shared by the token's routes
    // Tile mode of the batched kernel: blockIdx.y is a tile of pairs of one expert, taken from a
    // route plan (expert_bounds / tile_bounds / pair_order of mfqb_moe_route_plan).
    const int* expert_bounds;
    const int* tile_bounds;
    const int* pair_order;
    int n_experts;
    int private_sums;        // single-row kernel: one copy of the partial sums per warp instead of shared-memory atomics
    // Single-row kernel, row-parallel product: when reduce.world > 0 the CTA's summed rows are this
    // rank's partial result; they go to the peers and the sum over ranks is written to y.
    PeerReduce reduce;
    // Single-row kernel, expert FFN: x_mode 1 reads x as float32 [rows, k]; x_mode 2 reads the gate|up
    // products of the pair, float32 [pairs, 2k] (gate columns first), and forms the SwiGLU activation
    // up * gate / (1 + exp(-gate)) while loading (mfq/kernels/cuda/glu.cuh:6-17) -- the activation is
    // never stored.  With route_w set, the routed product also ends the FFN: a CTA writes its rows to
    // pair_out [pairs, ldy] float32, and the last of a token's `routes` CTAs to arrive adds them with
    // the route weights, in route order, into y_final [tokens, ldy] (moe_weighted_reduce,
    // mfq/kernels/cuda/moe.cu:2957-2977).  token_count: [tokens * gridDim.x] zeros, left zero again.
    // f16 batched kernel (nint_gemvh_bl.cuh): the scaled f16 activations in fragment order (x_frag_kernel), the
    // distance between tiles in 8-byte units, and the inverse scale of every source row.
    const uint2* x16f;
    size_t x16f_tile_stride;
    const float* x16_scale;
    int x_mode;
    // Single-row kernel, x_mode 3 (residual add + RMSNorm fused into the product): x is the float32 residual row h [k];
    // the product is taken with (h + norm_delta) / rms(h + norm_delta) * norm_gamma, and CTA 0 writes h + norm_delta to
    // norm_h_out (a buffer other than x) when that is not null.  norm_delta may be null.
    const float* norm_delta;
    const float* norm_gamma;
    float* norm_h_out;
    float norm_eps;
    // Single-row kernel, gated FFN: the weight's 16-row blocks alternate (gate rows, up rows); the kernel
    // writes up * silu(gate), n / 2 values, instead of the n products.
    int glu;
    const float* route_w;
    float* pair_out;
    unsigned* token_count;
    void* y_final;
    int y_final_dtype;
    // Batched kernel: the activation rows already quantised by x_planes_kernel, row r at
    // xq_g + r * ngp * QS and gtab_g + r * ngp (ngp = nchunks * 8 groups, QS quads per group).
    const uint2* xq_g;
    const float2* gtab_g;
};

__device__ __forceinline__ void pdl_launch_dependents_b() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait_b() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

__device__ __forceinline__ void cp_async16_b(void* smem_dst, const void* gsrc) {
    const unsigned d = (unsigned)__cvta_generic_to_shared(smem_dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(d), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cp_async_commit_b() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }

// D (s32) += A (u8, 16x32) * B (u8 or s8, 32x8)
__device__ __forceinline__ void imma_u8u8(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.u8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void imma_u8s8(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ void imma_s8u8(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.u8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void imma_s8s8(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// low plane (unsigned activations bytes) / high plane (signed), A signed or unsigned
template <bool A_SIGNED>
__device__ __forceinline__ void imma_planes(int (&dlo)[4], int (&dhi)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t lo0,
                                            uint32_t lo1, uint32_t hi0, uint32_t hi1) {
    if constexpr (A_SIGNED) {
        imma_s8u8(dlo, a0, a1, a2, a3, lo0, lo1);
        imma_s8s8(dhi, a0, a1, a2, a3, hi0, hi1);
    } else {
        imma_u8u8(dlo, a0, a1, a2, a3, lo0, lo1);
        imma_u8s8(dhi, a0, a1, a2, a3, hi0, hi1);
    }
}

// ---- weight codecs -------------------------------------------------------------------------------
// A codec tells the kernels how one lane's words of a record become tensor-core A registers and
// float scales.  Interface:
//   T (octets per group), WC (code words per lane), SW (scale words per lane), A_SIGNED, HAS_MIN,
//   NEEDS_OWN_SCALE (areg reads the lane's own scale words), MIN_CTAS (launch bound);
//   Ctx: per-CTA context; ctx_bytes(w) bytes at the start of dynamic shared memory, init() fills them;
//   areg(qw, r, ctx, own_sw): register r = ((f*T + t)*4 + a) of the lane's stream;
//   scales(sw, ctx, ss, sm): the four sub-scales / sub-mins of a lane's scale words, in the order
//   (row lo, group even), (lo, odd), (hi, even), (hi, odd).
template <int BITS, int T_>
struct NintCodec {
    static constexpr int T = T_;
    using BU = ByteUnit<BITS>;
    static constexpr int WC = BU::words_for(8 * T), SW = 2;
    static constexpr bool A_SIGNED = false, HAS_MIN = true, NEEDS_OWN_SCALE = false;
    static constexpr bool PLAIN_FORM = true;   // plain products take the stripped kernels (see gemv1_bl_kernel)
    static constexpr int QMID = 1 << (BITS - 1);   // centre of the code range (the f16 kernel decodes d * (q - QMID) - (m - d * QMID))
    static constexpr int MIN_CTAS = WC > 48 ? 1 : (WC > 24 ? 2 : 3);
    struct Ctx {
        __device__ __forceinline__ void init(unsigned char*, const NintDevB&, int, int) {}
    };
    __host__ __device__ static size_t ctx_bytes(const NintDevB&) { return 0; }
    __device__ static __forceinline__ uint32_t areg(const uint32_t* qw, int r, const Ctx&, const uint32_t*) { return BU::at(qw, r); }
    __device__ static __forceinline__ void scales(const uint32_t* sw, const Ctx&, float (&ss)[4], float (&sm)[4]) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            ss[i] = (float)((sw[0] >> (8 * i)) & 0xFF);
            sm[i] = (float)((sw[1] >> (8 * i)) & 0xFF);
        }
    }
};

// Split of R row-blocks over g CTAs: every CTA gets R / g, the first R % g one more.  CTAs are
// handed to the SMs round robin, so the extra row-blocks land on distinct SMs instead of pairing up
// on one (which an even spread of the remainder over the block indices does).
__device__ __forceinline__ void split_row_blocks(int b, int g, int total, int& first, int& count) {
    const int base = total / g, extra = total % g;
    first = b * base + min(b, extra);
    count = base + (b < extra ? 1 : 0);
}

// Records per warp ring: about 6 KB of ring per warp, between 2 and 6 stages.
__host__ __device__ constexpr int gemv1_bl_stages(int rec_words) {
    return 6144 / (rec_words * 4) < 2 ? 2 : (6144 / (rec_words * 4) > 6 ? 6 : 6144 / (rec_words * 4));
}
// Quads (uint2: low-plane word, high-plane word) per group in the staged activation row: 2T
// quads, padded so that the eight groups a warp reads together start in distinct banks.
__host__ __device__ constexpr int gemv1_bl_qstride(int t8) { return (2 * t8) % 8 == 0 ? 2 * t8 + 1 : 2 * t8; }

// The group scales the kernels multiply integer sums by carry a factor 2^-24, and every output is
// multiplied by 2^24 once at the end: float(sum) * scale then stays finite for every finite bf16
// input (a sum reaches 2^23 and a scale 2^113 for magnitudes next to the bf16 maximum).  The price:
// groups whose largest magnitude is below 2^-88 keep fewer than 16 bits.
constexpr uint32_t kXScaleShift = 24u;
constexpr float kXScaleUndo = 16777216.f;   // 2^24

// Quantises groups [g0, g0 + ngroups) of one activation row into shared memory (ngroups a multiple
// of 8): xq[gl * QS + j] = (low bytes, high bytes) of the four slots 4j..4j+3 of group g0 + gl,
// gtab[gl] = (sx_g, sx_g * X_g).  Four threads per group; every thread of the CTA must call it.
template <int T, typename XT = __nv_bfloat16>
__device__ __forceinline__ void stage_x_planes(const XT* __restrict__ xrow, int k, int gs, int g0, int ngroups, uint2* xq,
                                               float2* gtab) {
    constexpr int QS = gemv1_bl_qstride(T);
    constexpr uint32_t SH = sizeof(XT) == 2 ? 0u : 1u;   // float32 rows: one bit of head-room (a magnitude could round up to 2^15)
    const bool vec_ok = sizeof(XT) == 2 && (reinterpret_cast<uintptr_t>(xrow) & 7) == 0;
    for (int u = threadIdx.x; u < ngroups * 4; u += blockDim.x) {
        const int gl = u >> 2, g = g0 + gl, c = u & 3;
        float v[(2 * T + 3) / 4][4];
        uint32_t ab = 0u;   // largest magnitude of the group as float bits (orders like the value; NaN is largest)
#pragma unroll
        for (int jj = 0; jj < (2 * T + 3) / 4; ++jj) {
            const int j = c + 4 * jj, k0 = g * gs + 4 * j;
#pragma unroll
            for (int i = 0; i < 4; ++i) v[jj][i] = 0.f;
            if (j < 2 * T && 4 * j < gs) {
                if (vec_ok && (k0 & 3) == 0 && k0 + 3 < k && 4 * j + 3 < gs) {
                    const uint2 raw = __ldg(reinterpret_cast<const uint2*>(xrow + k0));
                    v[jj][0] = __uint_as_float(raw.x << 16);
                    v[jj][1] = __uint_as_float(raw.x & 0xFFFF0000u);
                    v[jj][2] = __uint_as_float(raw.y << 16);
                    v[jj][3] = __uint_as_float(raw.y & 0xFFFF0000u);
                } else {
#pragma unroll
                    for (int i = 0; i < 4; ++i)
                        if (4 * j + i < gs && k0 + i < k) v[jj][i] = (float)xrow[k0 + i];
                }
            }
#pragma unroll
            for (int i = 0; i < 4; ++i) ab = max(ab, __float_as_uint(v[jj][i]) & 0x7FFFFFFFu);
        }
        ab = max(ab, __shfl_xor_sync(0xffffffffu, ab, 1));
        ab = max(ab, __shfl_xor_sync(0xffffffffu, ab, 2));
        const uint32_t eb = max(ab >> 23, 15u + kXScaleShift);
        // eb = 255: an infinity or NaN in the group; its scale becomes NaN and so does every output
        const float sx = __uint_as_float(eb >= 255u ? 0x7FC00000u : (eb - 14u - kXScaleShift + SH) << 23);
        const float inv = __uint_as_float((268u - SH - min(eb, 254u)) << 23);
        constexpr float kMagic = 12582912.f;   // 1.5 * 2^23: the low 16 mantissa bits hold round(x * inv) in two's complement
        float xs = 0.f;
#pragma unroll
        for (int jj = 0; jj < (2 * T + 3) / 4; ++jj) {
            const int j = c + 4 * jj;
            uint32_t f[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float r = fmaf(v[jj][i], inv, kMagic);
                xs += r - kMagic;
                f[i] = __float_as_uint(r);
            }
            const uint32_t t01 = __byte_perm(f[0], f[1], 0x5140), t23 = __byte_perm(f[2], f[3], 0x5140);
            if (j < 2 * T) xq[gl * QS + j] = make_uint2(__byte_perm(t01, t23, 0x5410), __byte_perm(t01, t23, 0x7632));
        }
        xs += __shfl_xor_sync(0xffffffffu, xs, 1);
        xs += __shfl_xor_sync(0xffffffffu, xs, 2);
        if (c == 0) gtab[gl] = make_float2(sx, sx * xs);
    }
}

// Per-warp form for the single-row kernel: the warp quantises the eight groups of one chunk in
// registers.  Lane 4g + c loads quads c, c + 4, ... of group g (x_chunk_load), then x_chunk_quant
// returns what the lane feeds to the tensor core for its column (= group g): the byte planes of
// quads 2t + (c & 1), t = 0..T-1 -- its own quads and those of lane c ^ 2 -- and the (scale,
// scaled sum) pairs of groups 2c and 2c + 1.
template <int T>
struct XChunkRaw {
    static constexpr int JJ = (2 * T + 3) / 4;
    uint2 v[JJ];   // four bf16 each
};
template <int T>
__device__ __forceinline__ void x_chunk_load(const __nv_bfloat16* __restrict__ xrow, bool fast, bool vec_ok, int k, int gs, int g, int c,
                                             XChunkRaw<T>& raw) {
    if (fast) {   // the whole chunk lies inside the row, groups are whole quads, 8-byte loads are aligned
#pragma unroll
        for (int jj = 0; jj < XChunkRaw<T>::JJ; ++jj) {
            const int j = c + 4 * jj;
            raw.v[jj] = make_uint2(0u, 0u);
            if (j < 2 * T) raw.v[jj] = __ldg(reinterpret_cast<const uint2*>(xrow + g * gs + 4 * j));
        }
        return;
    }
#pragma unroll
    for (int jj = 0; jj < XChunkRaw<T>::JJ; ++jj) {
        const int j = c + 4 * jj, k0 = g * gs + 4 * j;
        raw.v[jj] = make_uint2(0u, 0u);
        if (j < 2 * T && 4 * j < gs) {
            if (vec_ok && (k0 & 3) == 0 && k0 + 3 < k && 4 * j + 3 < gs) {
                raw.v[jj] = __ldg(reinterpret_cast<const uint2*>(xrow + k0));
            } else {
                const unsigned short* xb = reinterpret_cast<const unsigned short*>(xrow);
                uint32_t e[4] = {0u, 0u, 0u, 0u};
#pragma unroll
                for (int i = 0; i < 4; ++i)
                    if (4 * j + i < gs && k0 + i < k) e[i] = __ldg(xb + k0 + i);
                raw.v[jj] = make_uint2(e[0] | (e[1] << 16), e[2] | (e[3] << 16));
            }
        }
    }
}
template <int T>
__device__ __forceinline__ void x_chunk_quant(const XChunkRaw<T>& raw, int c, uint32_t (&xlo)[T], uint32_t (&xhi)[T], float4& gt) {
    constexpr int JJ = XChunkRaw<T>::JJ;
    // largest magnitude of the group from the bf16 bit patterns (they order like the values; NaN is largest)
    uint32_t m2 = 0u;
#pragma unroll
    for (int jj = 0; jj < JJ; ++jj)
        m2 = __vimax3_s16x2(m2, raw.v[jj].x & 0x7FFF7FFFu, raw.v[jj].y & 0x7FFF7FFFu);
    uint32_t ab = max(m2 & 0xFFFFu, m2 >> 16);
    ab = max(ab, __shfl_xor_sync(0xffffffffu, ab, 1));
    ab = max(ab, __shfl_xor_sync(0xffffffffu, ab, 2));
    const uint32_t eb = max(ab >> 7, 15u + kXScaleShift);
    const float sx = __uint_as_float(eb >= 255u ? 0x7FC00000u : (eb - 14u - kXScaleShift) << 23);   // NaN for a group holding inf or NaN
    const float inv = __uint_as_float((268u - min(eb, 254u)) << 23);
    constexpr float kMagic = 12582912.f;   // 1.5 * 2^23
    uint32_t mine_lo[JJ], mine_hi[JJ];
    int xsum_lo = 0, xsum_hi = 0;
#pragma unroll
    for (int jj = 0; jj < JJ; ++jj) {
        const uint32_t f0 = __float_as_uint(fmaf(__uint_as_float(raw.v[jj].x << 16), inv, kMagic));
        const uint32_t f1 = __float_as_uint(fmaf(__uint_as_float(raw.v[jj].x & 0xFFFF0000u), inv, kMagic));
        const uint32_t f2 = __float_as_uint(fmaf(__uint_as_float(raw.v[jj].y << 16), inv, kMagic));
        const uint32_t f3 = __float_as_uint(fmaf(__uint_as_float(raw.v[jj].y & 0xFFFF0000u), inv, kMagic));
        const uint32_t t01 = __byte_perm(f0, f1, 0x5140), t23 = __byte_perm(f2, f3, 0x5140);
        mine_lo[jj] = __byte_perm(t01, t23, 0x5410);
        mine_hi[jj] = __byte_perm(t01, t23, 0x7632);
        xsum_lo = (int)__dp4a(mine_lo[jj], 0x01010101u, (unsigned)xsum_lo);   // unsigned low bytes
        xsum_hi = __dp4a((int)mine_hi[jj], 0x01010101, xsum_hi);              // signed high bytes
    }
    int xsi = xsum_hi * 256 + xsum_lo;   // sum of the lane's xi
    xsi += __shfl_xor_sync(0xffffffffu, xsi, 1);
    xsi += __shfl_xor_sync(0xffffffffu, xsi, 2);
    const float sxx = sx * (float)xsi;
    // quad 2t + (c&1) belongs to this lane when (t & 1) == (c >> 1), else to lane c ^ 2; either way slot t >> 1
    const bool own_even = (c >> 1) == 0;
#pragma unroll
    for (int jj = 0; jj < JJ; ++jj) {
        const uint32_t other_lo = __shfl_xor_sync(0xffffffffu, mine_lo[jj], 2), other_hi = __shfl_xor_sync(0xffffffffu, mine_hi[jj], 2);
        if (2 * jj < T) {
            xlo[2 * jj] = own_even ? mine_lo[jj] : other_lo;
            xhi[2 * jj] = own_even ? mine_hi[jj] : other_hi;
        }
        if (2 * jj + 1 < T) {
            xlo[2 * jj + 1] = own_even ? other_lo : mine_lo[jj];
            xhi[2 * jj + 1] = own_even ? other_hi : mine_hi[jj];
        }
    }
    gt.x = __shfl_sync(0xffffffffu, sx, 8 * c);
    gt.y = __shfl_sync(0xffffffffu, sxx, 8 * c);
    gt.z = __shfl_sync(0xffffffffu, sx, 8 * c + 4);
    gt.w = __shfl_sync(0xffffffffu, sxx, 8 * c + 4);
}

// Float32 forms of the two functions above (x_mode 1, 2 and 3).  A float32 magnitude could round up to
// 2^15 on the 16-bit grid, so these groups get one bit of head-room.
template <int T>
struct XChunkRawF {
    static constexpr int JJ = (2 * T + 3) / 4;
    float v[JJ][4];
};
template <int T, int XMODE>
__device__ __forceinline__ void x_chunk_load_f(const float* __restrict__ xrow, int k, int gs, int g, int c, XChunkRawF<T>& raw) {
    const bool vec_ok = (reinterpret_cast<uintptr_t>(xrow) & 15) == 0 && (gs & 3) == 0 && (k & 3) == 0;
#pragma unroll
    for (int jj = 0; jj < XChunkRawF<T>::JJ; ++jj) {
        const int j = c + 4 * jj, k0 = g * gs + 4 * j;
#pragma unroll
        for (int i = 0; i < 4; ++i) raw.v[jj][i] = 0.f;
        if (j < 2 * T && 4 * j < gs && k0 < k) {
            float a[4] = {0.f, 0.f, 0.f, 0.f}, u[4] = {1.f, 1.f, 1.f, 1.f};
            if (vec_ok && k0 + 3 < k) {
                // mode 3 reads the normalised row the CTA prepared in shared memory: no read-only global path there
                const float4 va = XMODE == 3 ? *reinterpret_cast<const float4*>(xrow + k0) : __ldg(reinterpret_cast<const float4*>(xrow + k0));
                a[0] = va.x; a[1] = va.y; a[2] = va.z; a[3] = va.w;
                if constexpr (XMODE == 2) {
                    const float4 vu = __ldg(reinterpret_cast<const float4*>(xrow + k + k0));
                    u[0] = vu.x; u[1] = vu.y; u[2] = vu.z; u[3] = vu.w;
                }
            } else {
#pragma unroll
                for (int i = 0; i < 4; ++i)
                    if (4 * j + i < gs && k0 + i < k) {
                        a[i] = XMODE == 3 ? xrow[k0 + i] : __ldg(xrow + k0 + i);
                        if constexpr (XMODE == 2) u[i] = __ldg(xrow + k + k0 + i);
                    }
            }
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                if constexpr (XMODE == 2) raw.v[jj][i] = u[i] * a[i] / (1.0f + expf(-a[i]));
                else raw.v[jj][i] = a[i];
            }
        }
    }
}
template <int T>
__device__ __forceinline__ void x_chunk_quant_f(const XChunkRawF<T>& raw, int c, uint32_t (&xlo)[T], uint32_t (&xhi)[T], float4& gt) {
    constexpr int JJ = XChunkRawF<T>::JJ;
    uint32_t ab = 0u;   // largest magnitude of the group as float bits (NaN is largest)
#pragma unroll
    for (int jj = 0; jj < JJ; ++jj)
#pragma unroll
        for (int i = 0; i < 4; ++i) ab = max(ab, __float_as_uint(raw.v[jj][i]) & 0x7FFFFFFFu);
    ab = max(ab, __shfl_xor_sync(0xffffffffu, ab, 1));
    ab = max(ab, __shfl_xor_sync(0xffffffffu, ab, 2));
    const uint32_t eb = max(ab >> 23, 15u + kXScaleShift);
    const float sx = __uint_as_float(eb >= 255u ? 0x7FC00000u : (eb - 13u - kXScaleShift) << 23);   // NaN for a group holding inf or NaN
    const float inv = __uint_as_float((267u - min(eb, 254u)) << 23);
    constexpr float kMagic = 12582912.f;   // 1.5 * 2^23
    uint32_t mine_lo[JJ], mine_hi[JJ];
    int xsum_lo = 0, xsum_hi = 0;
#pragma unroll
    for (int jj = 0; jj < JJ; ++jj) {
        const uint32_t f0 = __float_as_uint(fmaf(raw.v[jj][0], inv, kMagic)), f1 = __float_as_uint(fmaf(raw.v[jj][1], inv, kMagic));
        const uint32_t f2 = __float_as_uint(fmaf(raw.v[jj][2], inv, kMagic)), f3 = __float_as_uint(fmaf(raw.v[jj][3], inv, kMagic));
        const uint32_t t01 = __byte_perm(f0, f1, 0x5140), t23 = __byte_perm(f2, f3, 0x5140);
        mine_lo[jj] = __byte_perm(t01, t23, 0x5410);
        mine_hi[jj] = __byte_perm(t01, t23, 0x7632);
        xsum_lo = (int)__dp4a(mine_lo[jj], 0x01010101u, (unsigned)xsum_lo);
        xsum_hi = __dp4a((int)mine_hi[jj], 0x01010101, xsum_hi);
    }
    int xsi = xsum_hi * 256 + xsum_lo;
    xsi += __shfl_xor_sync(0xffffffffu, xsi, 1);
    xsi += __shfl_xor_sync(0xffffffffu, xsi, 2);
    const float sxx = sx * (float)xsi;
    const bool own_even = (c >> 1) == 0;
#pragma unroll
    for (int jj = 0; jj < JJ; ++jj) {
        const uint32_t other_lo = __shfl_xor_sync(0xffffffffu, mine_lo[jj], 2), other_hi = __shfl_xor_sync(0xffffffffu, mine_hi[jj], 2);
        if (2 * jj < T) {
            xlo[2 * jj] = own_even ? mine_lo[jj] : other_lo;
            xhi[2 * jj] = own_even ? mine_hi[jj] : other_hi;
        }
        if (2 * jj + 1 < T) {
            xlo[2 * jj + 1] = own_even ? other_lo : mine_lo[jj];
            xhi[2 * jj + 1] = own_even ? other_hi : mine_hi[jj];
        }
    }
    gt.x = __shfl_sync(0xffffffffu, sx, 8 * c);
    gt.y = __shfl_sync(0xffffffffu, sxx, 8 * c);
    gt.z = __shfl_sync(0xffffffffu, sx, 8 * c + 4);
    gt.w = __shfl_sync(0xffffffffu, sxx, 8 * c + 4);
}

// Routed product that also ends the expert FFN (GemvArgsB::route_w): this CTA's rows of its pair are in
// pair_out; the last of the token's CTAs with this block index adds the token's routes and writes y_final.
__device__ __forceinline__ void routed_finish_token(const GemvArgsB& a, int pair, int rbl0, int nrb, int row_limit) {
    __shared__ unsigned s_old;
    const int token = pair / a.routes;
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) s_old = atomicAdd(a.token_count + (size_t)token * gridDim.x + blockIdx.x, 1u);
    __syncthreads();
    if (s_old != (unsigned)(a.routes - 1)) return;
    __threadfence();
    for (int i = threadIdx.x; i < nrb * 16; i += blockDim.x) {
        const int row = rbl0 * 16 + i;
        if (row < row_limit) {
            float acc = 0.f;
            for (int r = 0; r < a.routes; ++r)
                acc += __ldg(a.route_w + (size_t)token * a.routes + r) * __ldcg(a.pair_out + ((size_t)token * a.routes + r) * a.ldy + row);
            if (a.y_final_dtype == 0 /* MFQB_F32 */) reinterpret_cast<float*>(a.y_final)[(size_t)token * a.ldy + row] = acc;
            else reinterpret_cast<__nv_bfloat16*>(a.y_final)[(size_t)token * a.ldy + row] = __float2bfloat16_rn(acc);
        }
    }
    if (threadIdx.x == 0) a.token_count[(size_t)token * gridDim.x + blockIdx.x] = 0u;
}
// The same for a CTA whose pair's expert is not held here (expert-parallel shard): its rows count as zeros.
__device__ __forceinline__ void routed_absent_pair(const GemvArgsB& a, int pair) {
    int rbl0, nrb;
    split_row_blocks(blockIdx.x, gridDim.x, a.rb_per_expert, rbl0, nrb);
    for (int i = threadIdx.x; i < nrb * 16; i += blockDim.x) {
        const int row = rbl0 * 16 + i;
        if (row < a.ldy) a.pair_out[(size_t)pair * a.ldy + row] = 0.f;
    }
    routed_finish_token(a, pair, rbl0, nrb, a.ldy);
}

// Shared memory: partial sums [warps or 1][rb_per_cta][16] f32 | anchors [rb_per_cta][16] u32 |
// per warp a ring of S item records.  With few row-blocks per CTA every warp adds into its own
// copy of the partial sums (plain read-modify-write), else all share one through atomics.  Every warp streams its own items (chunk-major) through its ring with
// 16-byte asynchronous copies; the first S items are requested before the kernel waits for its
// predecessor in the stream, since weights are constants.  The activation row is read straight
// from global memory, one chunk ahead, and quantised in registers by the warp that needs it.
// DENSE: the kernel serves plain products only (no routing table, no route sum, every warp its own chunks);
// the routed launches of the expert path compile the general form.
// PLAIN_OUT: no sum over ranks and no gated epilogue (the rows, or the routed pair's rows, are written as they are).
// ONE_RB (with PLAIN_OUT): the grid has one CTA per row-block (the 4096-row matrices): CTA b owns row-block b.
template <class C, int XMODE = 0, bool DENSE = false, bool PLAIN_OUT = false, bool ONE_RB = false>
__device__ __forceinline__ void gemv1_bl_body(const GemvArgsB& a, const NintDevB& w, unsigned char* smem) {
    constexpr int G = kChunkGroupsB, T = C::T, WC = C::WC, SW = C::SW, REC = (WC + SW) * 32;
    constexpr int S = gemv1_bl_stages(REC);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarps = blockDim.x >> 5;
    const int q = lane >> 2, c = lane & 3;
    typename C::Ctx ctx;
    ctx.init(smem, w, tid, blockDim.x);   // constant tables: visible after the first __syncthreads
    float* ypart = reinterpret_cast<float*>(smem + C::ctx_bytes(w));
    const int ycopies = a.private_sums ? nwarps : 1, ystride = a.rb_per_cta * 16;
    uint32_t* anch = reinterpret_cast<uint32_t*>(ypart + (size_t)ycopies * ystride);
    uint32_t* ring = anch + (size_t)a.rb_per_cta * 16 + (size_t)warp * S * REC;   // ctx_bytes is a multiple of 16

    // split of the row-blocks over gridDim.x (split_row_blocks): CTA b owns a contiguous range of the
    // R row-blocks of the whole matrix, or of its pair's expert in routed mode
    int rb_base = 0, rb_total = w.nrb;
    const __nv_bfloat16* xrow = a.x;
    size_t y_off = 0;
    const bool routed = !DENSE && a.route_ids != nullptr;
    if (routed) {
        pdl_wait_b();   // the routing table comes from the previous kernel
        const int pair = blockIdx.y, e = a.route_ids[pair];
        if (e < 0 || a.expert_pool[e] != a.pool) return;
        rb_total = a.rb_per_expert;
        rb_base = a.expert_local[e] * a.rb_per_expert;
        if constexpr (XMODE == 0) xrow += (size_t)(a.x_per_pair ? pair : pair / a.routes) * w.k;
        y_off = (size_t)pair * a.ldy;
    }
    int rbl0, nrb;
    if constexpr (ONE_RB) {
        rbl0 = blockIdx.x;
        nrb = 1;
    } else if (!PLAIN_OUT && a.glu) {   // whole (gate, up) pairs of row-blocks per CTA
        split_row_blocks(blockIdx.x, gridDim.x, rb_total >> 1, rbl0, nrb);
        rbl0 *= 2;
        nrb *= 2;
    } else {
        split_row_blocks(blockIdx.x, gridDim.x, rb_total, rbl0, nrb);
    }
    const int rb0 = rb_base + rbl0;
    const int row_limit = routed ? a.ldy : w.n;   // rows this problem has (an expert's rows are padded to whole blocks)

    // items of this warp, chunk-major: chunk = seg0, seg0 + cw, ...; inside a chunk the row-blocks
    // rg, rg + rgroups, ... of the CTA.  Rows with at least as many chunks as the CTA has warps give every
    // warp its own chunks and all row-blocks (cw = nwarps, one group); shorter rows (an expert's down
    // projection) split the warps into groups that share the chunks and take the row-blocks in turn.
    // Two cursors walk the sequence (issue runs S items ahead).
    int cw = nwarps, rgroups = 1, seg0 = warp, rg = 0;
    int my_segs, my_rbs = nrb;
    if (!DENSE && w.nchunks < nwarps) {   // every warp of a group has one chunk
        cw = w.nchunks;
        rgroups = nwarps / cw;
        rg = warp / cw;
        seg0 = warp - rg * cw;
        my_segs = rg < rgroups ? 1 : 0;
        my_rbs = rg < min(rgroups, nrb) ? (nrb - rg + rgroups - 1) / rgroups : 0;
    } else {
        my_segs = (w.nchunks - warp + nwarps - 1) / nwarps;
    }
    const int n_mine = my_segs * my_rbs;
    // the record pointer walks (chunk, row-block) incrementally: the warp's next row-block, or back to
    // its first row-block of its next chunk
    int iss_i = 0, iss_rbl = 0, iss_stage = 0;
    const uint32_t* iss_src = w.items + ((size_t)(rb0 + rg) * w.nchunks + seg0) * REC + lane * 4;
    const long long step_rb = (long long)rgroups * w.nchunks * REC, step_seg = (long long)cw * REC - (long long)(my_rbs - 1) * step_rb;
    auto issue = [&]() {
        if (iss_i < n_mine) {
            uint32_t* dst = ring + iss_stage * REC + lane * 4;
#pragma unroll
            for (int off = 0; off < REC; off += 128)
                if (off + 128 <= REC || lane * 4 < REC - off) cp_async16_b(dst + off, iss_src + off);
        }
        cp_async_commit_b();   // one group per item slot, empty past the end: keeps the wait count uniform
        ++iss_i;
        if (++iss_rbl == my_rbs) { iss_rbl = 0; iss_src += step_seg; }
        else iss_src += step_rb;
        if (++iss_stage == S) iss_stage = 0;
    };

    pdl_launch_dependents_b();
#pragma unroll
    for (int i = 0; i < S; ++i) issue();
    for (int i = tid; i < ycopies * ystride; i += blockDim.x) ypart[i] = 0.f;
    for (int i = tid; i < nrb * 16; i += blockDim.x) anch[i] = __ldg(w.anchors + rb0 * 16 + i);
    __syncthreads();
    pdl_wait_b();

    // Block-diagonal B: lane (q, c) feeds column q = group q of the chunk, which is octet q&3 of
    // the steps of family q>>2; its bytes are live only where the fragment's k-range (octet c>>1
    // of b0, octet 2 + (c>>1) of b1) is that octet.
    const bool live = (c >> 1) == (q & 1);
    const uint32_t m00 = (live && (q >> 1) == 0) ? 0xFFFFFFFFu : 0u, m01 = (live && (q >> 1) == 1) ? 0xFFFFFFFFu : 0u;
    const uint32_t m10 = (live && (q >> 1) == 2) ? 0xFFFFFFFFu : 0u, m11 = (live && (q >> 1) == 3) ? 0xFFFFFFFFu : 0u;

    const bool vec_ok = (reinterpret_cast<uintptr_t>(xrow) & 7) == 0;
    const bool fast_ok = vec_ok && (w.gs & 7) == 0;   // then chunks that end inside the row load without per-element checks
    const int chunk_len = G * w.gs;
    float* ymine = ypart + (a.private_sums ? warp * ystride : 0);
    int cur_seg = -1;
    uint32_t xlo[T], xhi[T];
    float4 gt = make_float4(0.f, 0.f, 0.f, 0.f);   // (sx, sx*X) of groups 2c, 2c+1 of the chunk
    XChunkRaw<T> raw;                              // the activations of the warp's next chunk, requested one chunk ahead
    XChunkRawF<T> rawf;
    // float32 rows: [rows, k], or the pair's gate|up products [pairs, 2k]
    const float* xrow_f = nullptr;
    if constexpr (XMODE == 3) {
        // residual add + RMSNorm of the row, once per CTA, into shared memory behind the rings (k is a multiple of 4)
        __shared__ float norm_red[32];
        float* xs = reinterpret_cast<float*>(anch + (size_t)a.rb_per_cta * 16 + (size_t)nwarps * S * REC);
        const float4* h4 = reinterpret_cast<const float4*>(a.x);
        const float4* d4 = reinterpret_cast<const float4*>(a.norm_delta);
        const float4* g4 = reinterpret_cast<const float4*>(a.norm_gamma);
        float4* o4 = (blockIdx.x == 0 && a.norm_h_out != nullptr) ? reinterpret_cast<float4*>(a.norm_h_out) : nullptr;
        float ss = 0.f;
        for (int i = tid; i < (w.k >> 2); i += blockDim.x) {
            float4 v = h4[i];
            if (d4 != nullptr) {
                const float4 dv = d4[i];
                v.x += dv.x; v.y += dv.y; v.z += dv.z; v.w += dv.w;
            }
            reinterpret_cast<float4*>(xs)[i] = v;
            if (o4 != nullptr) o4[i] = v;
            ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
        }
        for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        if (lane == 0) norm_red[warp] = ss;
        __syncthreads();
        float tot = 0.f;
        for (int i = 0; i < nwarps; ++i) tot += norm_red[i];
        const float inv = rsqrtf(tot / (float)w.k + a.norm_eps);
        for (int i = tid; i < (w.k >> 2); i += blockDim.x) {
            float4 v = reinterpret_cast<float4*>(xs)[i];
            const float4 gv = __ldg(g4 + i);
            v.x *= inv * gv.x; v.y *= inv * gv.y; v.z *= inv * gv.z; v.w *= inv * gv.w;
            reinterpret_cast<float4*>(xs)[i] = v;
        }
        __syncthreads();
        xrow_f = xs;
    } else if constexpr (XMODE != 0) {
        const size_t xr = routed ? (size_t)(a.x_per_pair ? blockIdx.y : blockIdx.y / a.routes) : 0;
        xrow_f = reinterpret_cast<const float*>(a.x) + xr * (XMODE == 2 ? 2 : 1) * w.k;
    }
    if (n_mine > 0) {
        if constexpr (XMODE == 0) x_chunk_load<T>(xrow, fast_ok && (seg0 + 1) * chunk_len <= w.k, vec_ok, w.k, w.gs, seg0 * G + q, c, raw);
        else x_chunk_load_f<T, XMODE>(xrow_f, w.k, w.gs, seg0 * G + q, c, rawf);
    }

    int seg = seg0, rbl = rg, stage = 0;
    float sum_lo = 0.f, sum_hi = 0.f;
    for (int i = 0; i < n_mine; ++i) {
        if (seg != cur_seg) {
            cur_seg = seg;
            if constexpr (XMODE == 0) {
                x_chunk_quant<T>(raw, c, xlo, xhi, gt);
                if (seg + cw < w.nchunks)
                    x_chunk_load<T>(xrow, fast_ok && (seg + cw + 1) * chunk_len <= w.k, vec_ok, w.k, w.gs, (seg + cw) * G + q, c, raw);
            } else {
                x_chunk_quant_f<T>(rawf, c, xlo, xhi, gt);
                if (seg + cw < w.nchunks) x_chunk_load_f<T, XMODE>(xrow_f, w.k, w.gs, (seg + cw) * G + q, c, rawf);
            }
        }
        asm volatile("cp.async.wait_group %0;\n" ::"n"(S - 1) : "memory");
        __syncwarp();
        const uint32_t* rec = ring + stage * REC;
        uint32_t qw[WC];
#pragma unroll
        for (int j = 0; j < WC; ++j) qw[j] = rec[j * 32 + lane];
        uint32_t sw[SW];
#pragma unroll
        for (int j = 0; j < SW; ++j) sw[j] = rec[(WC + j) * 32 + lane];
        __syncwarp();          // every lane has read the stage before it is refilled
        issue();
        int dlo[4] = {0, 0, 0, 0}, dhi[4] = {0, 0, 0, 0};
#pragma unroll
        for (int f = 0; f < 2; ++f) {
#pragma unroll
            for (int t = 0; t < T; ++t) {
                const int r = (f * T + t) * 4;
                const uint32_t a0 = C::areg(qw, r, ctx, sw), a1 = C::areg(qw, r + 1, ctx, sw), a2 = C::areg(qw, r + 2, ctx, sw),
                               a3 = C::areg(qw, r + 3, ctx, sw);
                const uint32_t mb0 = f ? m10 : m00, mb1 = f ? m11 : m01;
                imma_planes<C::A_SIGNED>(dlo, dhi, a0, a1, a2, a3, xlo[t] & mb0, xlo[t] & mb1, xhi[t] & mb0, xhi[t] & mb1);
            }
        }
        // D = 256 * high + low: sums of q * xi for rows (q, q+8) x groups (2c, 2c+1)
        const float d0 = (float)(dhi[0] * 256 + dlo[0]) * gt.x, d1 = (float)(dhi[1] * 256 + dlo[1]) * gt.z;
        const float d2 = (float)(dhi[2] * 256 + dlo[2]) * gt.x, d3 = (float)(dhi[3] * 256 + dlo[3]) * gt.z;
        const uint32_t an_lo = anch[rbl * 16 + q], an_hi = anch[rbl * 16 + q + 8];
        const float2 f_lo = __half22float2(*reinterpret_cast<const __half2*>(&an_lo));   // (ns, nm)
        const float2 f_hi = __half22float2(*reinterpret_cast<const __half2*>(&an_hi));
        float ss[4], sm[4];
        C::scales(sw, ctx, ss, sm);
        float v_lo = f_lo.x * fmaf(ss[1], d1, ss[0] * d0), v_hi = f_hi.x * fmaf(ss[3], d3, ss[2] * d2);
        if constexpr (C::HAS_MIN) {
            v_lo -= f_lo.y * fmaf(sm[1], gt.w, sm[0] * gt.y);
            v_hi -= f_hi.y * fmaf(sm[3], gt.w, sm[2] * gt.y);
        }
        // the four lanes of a quad hold different groups of the same two rows
        v_lo += __shfl_xor_sync(0xffffffffu, v_lo, 1);
        v_hi += __shfl_xor_sync(0xffffffffu, v_hi, 1);
        v_lo += __shfl_xor_sync(0xffffffffu, v_lo, 2);
        v_hi += __shfl_xor_sync(0xffffffffu, v_hi, 2);
        if constexpr (ONE_RB) {   // one row-block: the warp's items add up in registers
            sum_lo += v_lo;
            sum_hi += v_hi;
        } else if (c == 0) {
            if (a.private_sums) {   // this warp's own copy: no other warp touches it
                ymine[rbl * 16 + q] += v_lo;
                ymine[rbl * 16 + q + 8] += v_hi;
            } else {
                atomicAdd(ypart + rbl * 16 + q, v_lo);
                atomicAdd(ypart + rbl * 16 + q + 8, v_hi);
            }
        }
        rbl += rgroups;
        if (rbl >= nrb) { rbl = rg; seg += cw; }
        if (++stage == S) stage = 0;
    }
    if constexpr (ONE_RB) {
        if (c == 0 && n_mine > 0) {   // the launch gives this form per-warp copies of the sums
            ymine[q] = sum_lo;
            ymine[q + 8] = sum_hi;
        }
    }
    asm volatile("cp.async.wait_group 0;\n" ::: "memory");
    __syncthreads();
    if (!PLAIN_OUT && a.reduce.world > 0) {
        // every thread owns one row of the CTA: it pushes this rank's partial value into slot `rank` of
        // every rank and sums the ranks' values of that row (the peers' CTAs with this block index
        // own the same rows: same shape, same grid)
        const PeerReduce& pr = a.reduce;
        const unsigned seq = peer_call_seq(pr);   // after griddepcontrol.wait: the previous call has published its number
        for (int i = tid; i < nrb * 16; i += blockDim.x) {
            const int row = rbl0 * 16 + i;
            if (row < row_limit) {
                float v = ypart[i];
                for (int cp = 1; cp < ycopies; ++cp) v += ypart[cp * ystride + i];
                peer_push(pr, seq, row, v * kXScaleUndo);
            }
        }
        for (int i = tid; i < nrb * 16; i += blockDim.x) {
            const int row = rbl0 * 16 + i;
            if (row < row_limit) {
                const float v = peer_sum(pr, seq, row, MFQB_ERR_TIMEOUT);
                if (a.y_dtype == 0 /* MFQB_F32 */) reinterpret_cast<float*>(a.y)[y_off + row] = v;
                else reinterpret_cast<__nv_bfloat16*>(a.y)[y_off + row] = __float2bfloat16_rn(v);
            }
        }
        peer_call_done(pr, seq);
        return;
    }
    if (!PLAIN_OUT && a.glu) {
        const int half = w.n >> 1;
        for (int i = tid; i < nrb * 8; i += blockDim.x) {
            const int pr = i >> 4, r = i & 15, row = (rbl0 >> 1) * 16 + i;
            if (row < half) {
                float g = ypart[pr * 32 + r], u = ypart[pr * 32 + 16 + r];
                for (int cp = 1; cp < ycopies; ++cp) {
                    g += ypart[cp * ystride + pr * 32 + r];
                    u += ypart[cp * ystride + pr * 32 + 16 + r];
                }
                g *= kXScaleUndo;
                u *= kXScaleUndo;
                const float v = u * g / (1.0f + expf(-g));
                if (a.y_dtype == 0 /* MFQB_F32 */) reinterpret_cast<float*>(a.y)[row] = v;
                else reinterpret_cast<__nv_bfloat16*>(a.y)[row] = __float2bfloat16_rn(v);
            }
        }
        return;
    }
    for (int i = tid; i < nrb * 16; i += blockDim.x) {
        const int row = rbl0 * 16 + i;   // row inside the problem (matrix, or the pair's expert)
        if (row < row_limit) {
            float v = ypart[i];
            for (int cp = 1; cp < ycopies; ++cp) v += ypart[cp * ystride + i];
            v *= kXScaleUndo;
            if (!DENSE && a.route_w != nullptr) a.pair_out[y_off + row] = v;
            else if (a.y_dtype == 0 /* MFQB_F32 */) reinterpret_cast<float*>(a.y)[y_off + row] = v;
            else reinterpret_cast<__nv_bfloat16*>(a.y)[y_off + row] = __float2bfloat16_rn(v);
        }
    }
    if (!DENSE && a.route_w != nullptr) routed_finish_token(a, blockIdx.y, rbl0, nrb, row_limit);
}

template <class C>
__global__ void __launch_bounds__(C::MIN_CTAS >= 3 ? 384 : 256, C::MIN_CTAS >= 3 ? 2 : C::MIN_CTAS) gemv1_bl_kernel(const GemvArgsB a) {
    extern __shared__ __align__(16) unsigned char smem[];
    gemv1_bl_body<C, 0, true, true>(a, a.w, smem);
}

// Residual add + RMSNorm fused into the product (x_mode 3; the gated epilogue may follow).
template <class C>
__global__ void __launch_bounds__(C::MIN_CTAS >= 3 ? 384 : 256, C::MIN_CTAS >= 3 ? 2 : C::MIN_CTAS) gemv1_bl_norm_kernel(const GemvArgsB a) {
    extern __shared__ __align__(16) unsigned char smem[];
    gemv1_bl_body<C, 3, true, false>(a, a.w, smem);
}

// One CTA per row-block (launched when the grid equals the number of row-blocks).
template <class C>
__global__ void __launch_bounds__(C::MIN_CTAS >= 3 ? 384 : 256, C::MIN_CTAS >= 3 ? 2 : C::MIN_CTAS) gemv1_bl_one_kernel(const GemvArgsB a) {
    extern __shared__ __align__(16) unsigned char smem[];
    gemv1_bl_body<C, 0, true, true, true>(a, a.w, smem);
}

// The same with the epilogues that do more than write the rows: the sum over ranks (row-parallel shards) and
// the gated activation over (gate, up) pairs of row-blocks.
template <class C>
__global__ void __launch_bounds__(C::MIN_CTAS >= 3 ? 384 : 256, C::MIN_CTAS >= 3 ? 2 : C::MIN_CTAS) gemv1_bl_epi_kernel(const GemvArgsB a) {
    extern __shared__ __align__(16) unsigned char smem[];
    gemv1_bl_body<C, 0, true, false>(a, a.w, smem);
}

// The general form for one cohort of an expert record: blockIdx.y is a (token, route) pair (per-cohort launches of
// records whose cohorts the all-cohort kernel does not hold).
template <class C>
__global__ void __launch_bounds__(C::MIN_CTAS >= 3 ? 384 : 256, C::MIN_CTAS >= 3 ? 2 : C::MIN_CTAS) gemv1_bl_routed_kernel(const GemvArgsB a) {
    extern __shared__ __align__(16) unsigned char smem[];
    gemv1_bl_body<C, 0, false>(a, a.w, smem);
}

// x is the float32 gate|up row [2k] of a gated FFN: the SwiGLU activation is computed as the row is
// loaded (x_chunk_load_f, mode 2), so the down projection needs no activation kernel before it.
template <class C>
__global__ void __launch_bounds__(C::MIN_CTAS >= 3 ? 384 : 256, C::MIN_CTAS >= 3 ? 2 : C::MIN_CTAS) gemv1_bl_swiglu_kernel(const GemvArgsB a) {
    extern __shared__ __align__(16) unsigned char smem[];
    gemv1_bl_body<C, 2, true>(a, a.w, smem);
}

// Several weights that share x, the code width, the group size and k (a.w describes their common
// geometry): blockIdx.y picks the weight, the CTAs of a row of the grid split its row-blocks.
template <class C>
__global__ void __launch_bounds__(C::MIN_CTAS >= 3 ? 384 : 256, C::MIN_CTAS >= 3 ? 2 : C::MIN_CTAS) gemv1_bl_multi_kernel(const GemvArgsB a, const __grid_constant__ GemvMultiTable table) {
    extern __shared__ __align__(16) unsigned char smem[];
    const GemvMultiEntry& e = table.e[blockIdx.y];
    if ((int)blockIdx.x >= e.nrb) return;   // fewer row-blocks than CTAs in this row of the grid
    GemvArgsB b = a;
    b.w.items = e.items;
    b.w.anchors = e.anchors;
    b.w.n = e.n;
    b.w.nrb = e.nrb;
    b.y = e.y;
    gemv1_bl_body<C, 0, true, true>(b, b.w, smem);
}

}  // namespace mfqb
