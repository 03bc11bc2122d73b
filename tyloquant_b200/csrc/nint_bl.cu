// Byte-lane NINT: decoder kernel and the launch planning of the GEMV kernels.
#include <algorithm>
#include <mutex>
#include <type_traits>

#include "common.h"
#include "cuda_util.h"
#include "nint_gemv_bl_launch.cuh"

namespace mfqb {

// ---- reference decoder on the GPU -----------------------------------------------------------
// One thread per (row, group, quad of four slots): reads its codes and the two scale bytes
// through the same accessors as the GEMV and writes w = fl(fl(d*q) - m), d = fl(ns*ss),
// m = fl(nm*sm): three separately rounded float32 operations, as the reference decoder does
// (mfq/quantize/nint_quant.py:896-908).
template <int BITS>
__global__ void nint_bl_dequant_kernel(const NintDevB w, void* out, int out_dtype) {
    using BU = ByteUnit<BITS>;
    const int quads = 2 * w.t8;
    const size_t total = (size_t)w.n * w.ng * quads;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
        const int j = (int)(idx % quads);
        const size_t rg = idx / quads;
        const int grp = (int)(rg % w.ng), row = (int)(rg / w.ng);
        if (4 * j >= w.gs) continue;
        const int rb = row >> 4, q = row & 7, hi = (row >> 3) & 1, ch = grp / kChunkGroupsB, g = grp % kChunkGroupsB;
        const int f = g >> 2, o = g & 3;
        const int lane = 4 * q + 2 * (o & 1) + (j & 1);
        const int reg = (f * w.t8 + (j >> 1)) * 4 + 2 * (o >> 1) + hi;
        const uint32_t* rec = w.items + ((size_t)rb * w.nchunks + ch) * w.rec_words;
        uint32_t uw[BU::U];
#pragma unroll
        for (int u = 0; u < BU::U; ++u) uw[u] = rec[((reg / BU::NP) * BU::U + u) * 32 + lane];
        const uint32_t codes = BU::at(uw, reg % BU::NP);
        const int slane = 4 * q + (g >> 1), sbyte = 8 * (2 * hi + (g & 1));
        const float ss = (float)((rec[w.wc * 32 + slane] >> sbyte) & 0xFF), sm = (float)((rec[(w.wc + 1) * 32 + slane] >> sbyte) & 0xFF);
        const uint32_t an = w.anchors[row];
        const float2 nsm = __half22float2(*reinterpret_cast<const __half2*>(&an));
        const float d = __fmul_rn(nsm.x, ss), m = __fmul_rn(nsm.y, sm);
        const int k0 = grp * w.gs + 4 * j;
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            if (4 * j + e < w.gs && k0 + e < w.k) {
                const float v = __fsub_rn(__fmul_rn(d, (float)((codes >> (8 * e)) & 0xFF)), m);
                const size_t off = (size_t)row * w.k + k0 + e;
                if (out_dtype == MFQB_F32) reinterpret_cast<float*>(out)[off] = v;
                else reinterpret_cast<__nv_bfloat16*>(out)[off] = __float2bfloat16_rn(v);
            }
        }
    }
}

void launch_nint_bl_dequant(const NintDevB& w, void* out, int out_dtype, cudaStream_t s) {
    const size_t total = (size_t)w.n * w.ng * 2 * w.t8;
    const int block = 256;
    const int grid = (int)std::min<size_t>((total + block - 1) / block, 148 * 32);
    switch (w.bits) {
        case 2: nint_bl_dequant_kernel<2><<<grid, block, 0, s>>>(w, out, out_dtype); break;
        case 3: nint_bl_dequant_kernel<3><<<grid, block, 0, s>>>(w, out, out_dtype); break;
        case 4: nint_bl_dequant_kernel<4><<<grid, block, 0, s>>>(w, out, out_dtype); break;
        case 5: nint_bl_dequant_kernel<5><<<grid, block, 0, s>>>(w, out, out_dtype); break;
        case 6: nint_bl_dequant_kernel<6><<<grid, block, 0, s>>>(w, out, out_dtype); break;
        case 8: nint_bl_dequant_kernel<8><<<grid, block, 0, s>>>(w, out, out_dtype); break;
        default: fail(MFQB_ERR_UNSUPPORTED, "NINT%d has no kernel", w.bits);
    }
    MFQB_CUDA(cudaGetLastError());
}

bool nint_bl_supported(int bits, int gs) {
    const int t8 = (gs + 7) / 8;
    return gs >= 8 && gs <= 64 && nint_bl_in_catalog(bits, t8);
}

// ---- GEMV launch planning ---------------------------------------------------------------------
cudaError_t launch_gemv_bl_nvq(const GemvArgsB& a, const GemvPlanB& p, cudaStream_t stream);

static void dispatch(const GemvArgsB& a, const GemvPlanB& p, cudaStream_t s, const char* what) {
    cudaError_t e;
    switch (a.w.bits) {
        case 0: e = launch_gemv_bl_nvq(a, p, s); break;   // lattice records
        case 2: e = launch_gemv_bl_bits<2>(a, p, s); break;
        case 3: e = launch_gemv_bl_bits<3>(a, p, s); break;
        case 4: e = launch_gemv_bl_bits<4>(a, p, s); break;
        case 5: e = launch_gemv_bl_bits<5>(a, p, s); break;
        case 6: e = launch_gemv_bl_bits<6>(a, p, s); break;
        case 8: e = launch_gemv_bl_bits<8>(a, p, s); break;
        default: fail(MFQB_ERR_UNSUPPORTED, "NINT%d has no kernel", a.w.bits);
    }
    if (e != cudaSuccess)
        fail(MFQB_ERR_CUDA, "%s%d gs=%d %s launch: %s", a.w.bits ? "NINT" : "NVQ index bits ", a.w.bits ? a.w.bits : a.w.index_bits, a.w.gs, what,
             cudaGetErrorString(e));
}

constexpr size_t kGemvSmemLimit = 200 * 1024;

// Shared-memory tables of the record's codec (lattice records: signed table + state scales).
static size_t codec_ctx_bytes(const NintDevB& w) { return w.table ? (size_t)w.table_words * 4 + 64 : 0; }
// CTAs of `smem` bytes each that fit an SM, at most `cap`.
static int ctas_per_sm(size_t smem, int cap) { return std::max(1, std::min(cap, (int)((220 * 1024) / (smem + 1024)))); }

// Per-warp copies of the partial sums while they stay small; shared copy with atomics beyond.
static bool gemv1_private_sums(int rb_per_cta) { return rb_per_cta <= 8; }
static size_t gemv1_smem(const NintDevB& w, int rb_per_cta, int warps) {
    const int copies = gemv1_private_sums(rb_per_cta) ? warps : 1;
    return codec_ctx_bytes(w) + (size_t)(copies + 1) * rb_per_cta * 16 * 4 + (size_t)warps * gemv1_bl_stages(w.rec_words) * w.rec_words * 4;
}
// Warps per CTA of the single-row kernel: each warp owns whole chunks of K, so 8 to 12 warps are
// chosen to make the largest number of chunks per warp as small as possible (wide records and the
// larger lattice codebooks stay at 8: their kernels are built for 256 threads).
static int gemv1_warps(const NintDevB& w) {
    if ((w.table && w.index_bits != 8) || w.wc > 24) return 8;
    int best = 8;
    for (int n = 9; n <= 12; ++n)
        if ((w.nchunks + n - 1) / n < (w.nchunks + best - 1) / best) best = n;
    return best;
}
static size_t gemvn_smem(const NintDevB& w, int rb_per_cta, int passes) {
    const int mb = 2 * passes;
    return codec_ctx_bytes(w) + (size_t)(mb + 1) * rb_per_cta * 16 * 4 + (size_t)8 * 2 * mb * gemvn_bl_row_bytes(w.t8) +
           (size_t)8 * gemvn_bl_stages(w.rec_words, passes) * w.rec_words * 4;
}

// Bytes of the quantised planes of `rows` activation rows for this weight.
size_t nint_bl_planes_bytes(const NintDevB& w, int rows) {
    return (size_t)rows * w.nchunks * kChunkGroupsB * (gemv1_bl_qstride(w.t8) + 1) * 8;
}

// Quantises x [rows, k] (bf16, or float32 when x_f32) into `planes` (nint_bl_planes_bytes): xq for all rows, then gtab.
void launch_x_planes(const NintDevB& w, const void* x, int rows, void* planes, const uint2** xq_g, const float2** gtab_g, cudaStream_t s,
                     bool x_f32) {
    const int ngp = w.nchunks * kChunkGroupsB, qs = gemv1_bl_qstride(w.t8);
    uint2* xq = static_cast<uint2*>(planes);
    float2* gtab = reinterpret_cast<float2*>(xq + (size_t)rows * ngp * qs);
    *xq_g = xq;
    *gtab_g = gtab;
    // 64 groups per CTA: one pass of its 256 threads (four threads per group)
    const dim3 grid((unsigned)((ngp + 63) / 64), (unsigned)rows);
    auto go = [&](auto t8) {
        constexpr int T = decltype(t8)::value;
        if (x_f32) x_planes_kernel<T, float><<<grid, 256, 0, s>>>(static_cast<const float*>(x), w.k, w.gs, ngp, 64, xq, gtab);
        else x_planes_kernel<T, __nv_bfloat16><<<grid, 256, 0, s>>>(static_cast<const __nv_bfloat16*>(x), w.k, w.gs, ngp, 64, xq, gtab);
    };
    switch (w.t8) {
        case 2: go(std::integral_constant<int, 2>{}); break;
        case 3: go(std::integral_constant<int, 3>{}); break;
        case 4: go(std::integral_constant<int, 4>{}); break;
        case 5: go(std::integral_constant<int, 5>{}); break;
        case 6: go(std::integral_constant<int, 6>{}); break;
        case 8: go(std::integral_constant<int, 8>{}); break;
        default: fail(MFQB_ERR_UNSUPPORTED, "group size %d has no kernel", w.gs);
    }
    MFQB_CUDA(cudaGetLastError());
}

// Library scratch for the planes of a plain batched product (per device, grow-only).
static void* planes_scratch(int device, size_t bytes, cudaStream_t s) {
    static GrowOnlyScratch pool;
    return pool.get(device, bytes, s, "mfqb_mul_mat (quantised activation planes)");
}

static int passes_for(int m) { return m <= 2 ? 1 : (m <= 4 ? 2 : 4); }

// This thread's share of the largest magnitude of a row, as float bits (they order like the values; NaN and
// infinity are largest): threads tid, tid + nthreads, ... take 16-byte pieces where the row is aligned.
__device__ __forceinline__ uint32_t row_absmax_part(const void* x, bool x_f32, size_t row, int k, int tid, int nthreads) {
    uint32_t ab = 0u;
    if (x_f32) {
        const float* p = static_cast<const float*>(x) + row * k;
        int j0 = 0;
        if ((reinterpret_cast<uintptr_t>(p) & 15) == 0) {
            const int nv = k >> 2;
#pragma unroll 4
            for (int j = tid; j < nv; j += nthreads) {
                const float4 v = __ldg(reinterpret_cast<const float4*>(p) + j);
                ab = max(max(ab, __float_as_uint(fabsf(v.x))), max(__float_as_uint(fabsf(v.y)), max(__float_as_uint(fabsf(v.z)), __float_as_uint(fabsf(v.w)))));
            }
            j0 = nv << 2;
        }
        for (int j = j0 + tid; j < k; j += nthreads) ab = max(ab, __float_as_uint(fabsf(p[j])));
    } else {
        const __nv_bfloat16* p = static_cast<const __nv_bfloat16*>(x) + row * k;
        int j0 = 0;
        if ((reinterpret_cast<uintptr_t>(p) & 15) == 0) {
            const int nv = k >> 3;
#pragma unroll 4
            for (int j = tid; j < nv; j += nthreads) {
                const uint4 v = __ldg(reinterpret_cast<const uint4*>(p) + j);
                const uint32_t w4[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                for (int i = 0; i < 4; ++i) ab = max(ab, max(w4[i] & 0x7FFF0000u, (w4[i] << 16) & 0x7FFF0000u));
            }
            j0 = nv << 3;
        }
        for (int j = j0 + tid; j < k; j += nthreads) ab = max(ab, __float_as_uint(fabsf(__bfloat162float(p[j]))));
    }
    return ab;
}
// (2^e, 2^-e) with 2^e * max in [2^14, 2^15); (1, 1) for a zero, subnormal or non-finite maximum.
__device__ __forceinline__ float2 row_scale_pair(uint32_t absmax_bits) {
    const int eb = (int)(absmax_bits >> 23);
    if (eb == 0 || eb == 255) return make_float2(1.f, 1.f);
    return make_float2(__uint_as_float((uint32_t)(127 + 14 - (eb - 127)) << 23), __uint_as_float((uint32_t)(127 - 14 + (eb - 127)) << 23));
}

// up[row] = 2^e with 2^e * max|x[row]| in [2^14, 2^15) (1 for a zero, subnormal or non-finite row), down[row] = 2^-e.
// One CTA of 1024 threads per row.
template <typename XT>
__global__ void __launch_bounds__(1024) x_row_scale_kernel(const XT* __restrict__ x, int k, float* __restrict__ up, float* __restrict__ down) {
    __shared__ uint32_t red[32];
    pdl_wait_b();
    pdl_launch_dependents_b();
    uint32_t ab = row_absmax_part(x, sizeof(XT) == 4, blockIdx.x, k, threadIdx.x, blockDim.x);
    for (int o = 16; o > 0; o >>= 1) ab = max(ab, __shfl_xor_sync(0xffffffffu, ab, o));
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ab;
    __syncthreads();
    ab = red[threadIdx.x & 31];
    for (int o = 16; o > 0; o >>= 1) ab = max(ab, __shfl_xor_sync(0xffffffffu, ab, o));
    if (threadIdx.x == 0) {
        const float2 sc = row_scale_pair(ab);
        up[blockIdx.x] = sc.x;
        down[blockIdx.x] = sc.y;
    }
}

// x_frag_kernel: see XFragArgs.
__global__ void __launch_bounds__(256) x_frag_kernel(const __grid_constant__ XFragArgs a) {
    __shared__ int rows_s[16];
    __shared__ float up_s[16];
    pdl_wait_b();
    pdl_launch_dependents_b();
    const int t = blockIdx.y, MB = 8 * a.nt;
    int pool = 0, m_cur = a.m, p0 = 0;
    if (a.tile_bounds != nullptr) {
        if (t >= a.tile_bounds[a.n_experts]) return;
        int lo = 0, hi = a.n_experts - 1;   // expert e with tile_bounds[e] <= t < tile_bounds[e + 1]
        while (lo < hi) {
            const int mid = (lo + hi + 1) >> 1;
            if (a.tile_bounds[mid] <= t) lo = mid;
            else hi = mid - 1;
        }
        pool = a.expert_pool[lo];
        if (pool < 0) return;
        p0 = a.expert_bounds[lo] + (t - a.tile_bounds[lo]) * MB;
        m_cur = min(MB, a.expert_bounds[lo + 1] - p0);
    }
    const int T = a.pool_t8[pool], seg = blockIdx.x;
    if (seg >= a.pool_nchunks[pool]) return;
    if (threadIdx.x < 16) {
        int r = -1;
        if ((int)threadIdx.x < m_cur) {
            if (a.tile_bounds != nullptr) {
                const int pair = a.pair_order[p0 + threadIdx.x];
                r = a.x_per_pair ? pair : pair / a.routes;
            } else {
                r = threadIdx.x;
            }
        }
        rows_s[threadIdx.x] = r;
        up_s[threadIdx.x] = r >= 0 ? a.up[r] : 0.f;
    }
    __syncthreads();
    uint2* dst = a.out + (size_t)t * a.tile_stride + (size_t)seg * 4 * T * a.nt * 32;
    for (int idx = threadIdx.x; idx < 4 * T * a.nt * 32; idx += blockDim.x) {
        const int lane = idx & 31, rest = idx >> 5, nt_i = rest % a.nt, j = rest / a.nt;
        const int h = j & 1, ft = j >> 1, f = ft / T, tt = ft - f * T;
        const int q = lane >> 2, c = lane & 3, r = rows_s[8 * nt_i + q];
        const int kk = seg * 64 * T + (4 * f + 2 * h + (c >> 1)) * 8 * T + 8 * tt + 4 * (c & 1);
        float v[4] = {0.f, 0.f, 0.f, 0.f};
        if (r >= 0) {
            const float up = up_s[8 * nt_i + q];
            const size_t e0 = (size_t)r * a.k + kk;
            if (!a.x_f32 && kk + 3 < a.k && ((reinterpret_cast<uintptr_t>(a.x) + e0 * 2) & 7) == 0) {   // the four bf16 in one load
                const uint2 w2 = __ldg(reinterpret_cast<const uint2*>(static_cast<const __nv_bfloat16*>(a.x) + e0));
                v[0] = __uint_as_float(w2.x << 16) * up;
                v[1] = __uint_as_float(w2.x & 0xFFFF0000u) * up;
                v[2] = __uint_as_float(w2.y << 16) * up;
                v[3] = __uint_as_float(w2.y & 0xFFFF0000u) * up;
            } else {
#pragma unroll
                for (int i = 0; i < 4; ++i)
                    if (kk + i < a.k)
                        v[i] = (a.x_f32 ? static_cast<const float*>(a.x)[e0 + i] : __bfloat162float(static_cast<const __nv_bfloat16*>(a.x)[e0 + i])) * up;
            }
        }
        __half hv[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) hv[i] = isfinite(v[i]) ? __float2half_rn(v[i]) : __ushort_as_half((unsigned short)0x7E00);   // non-finite input -> NaN
        uint2 pk;
        pk.x = (uint32_t)__half_as_ushort(hv[0]) | ((uint32_t)__half_as_ushort(hv[1]) << 16);
        pk.y = (uint32_t)__half_as_ushort(hv[2]) | ((uint32_t)__half_as_ushort(hv[3]) << 16);
        dst[idx] = pk;
    }
}

// ---- f16 batched kernel (nint_gemvh_bl.cuh) ------------------------------------------------------
// Needs group sizes that are whole octets (padded group sizes keep the integer kernels).
static size_t gemvh_smem(const NintDevB& w, int rb_per_cta, int nt) {
    const int mb = 8 * nt;
    return codec_ctx_bytes(w) + (size_t)(mb + 1) * rb_per_cta * 16 * 4 + (size_t)8 * gemvh_stages(w.rec_words) * w.rec_words * 4;
}
bool nint_bl_gemvh_supported(const NintDevB& w, int rows_per_launch) {
    // (lattice records stay on the integer kernels: measured, their table lookups leave the f16 form no gain)
    return !w.table && w.gs == 8 * w.t8 && gemvh_smem(w, 1, rows_per_launch > 8 ? 2 : 1) <= kGemvSmemLimit;
}
// 8-byte units of one tile (8 nt rows) of this weight's fragment-ordered activations.
size_t nint_bl_frag_tile_units(const NintDevB& w, int nt) { return (size_t)w.nchunks * 4 * w.t8 * nt * 32; }
// Bytes of the fragment buffer for `tiles` tiles of `tile_units` each plus the scales of `in_rows` source rows.
size_t x_frags_bytes(int in_rows, int tiles, size_t tile_units) { return ((size_t)tiles * tile_units * 8 + 255) / 256 * 256 + (size_t)in_rows * 8; }

// Row scales, then the fragments: fa carries the source rows, the tile description and the cohort geometry;
// `buf` is x_frags_bytes(in_rows, tiles, fa.tile_stride).  Returns the fragment base and the inverse row scales.
void launch_x_frags(XFragArgs fa, int in_rows, int tiles, int max_nchunks, void* buf, const uint2** xf, const float** down, cudaStream_t s) {
    uint2* frags = static_cast<uint2*>(buf);
    float* up = reinterpret_cast<float*>(static_cast<char*>(buf) + ((size_t)tiles * fa.tile_stride * 8 + 255) / 256 * 256);
    float* dn = up + in_rows;
    // both launched as programmatic dependents: they become resident while the previous kernel drains and wait
    // for it (the previous product may still read this buffer) before they touch memory
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)in_rows);
    cfg.blockDim = dim3(1024);
    cfg.stream = s;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (fa.x_f32) MFQB_CUDA(cudaLaunchKernelEx(&cfg, x_row_scale_kernel<float>, static_cast<const float*>(fa.x), fa.k, up, dn));
    else MFQB_CUDA(cudaLaunchKernelEx(&cfg, x_row_scale_kernel<__nv_bfloat16>, static_cast<const __nv_bfloat16*>(fa.x), fa.k, up, dn));
    fa.up = up;
    fa.out = frags;
    cfg.gridDim = dim3((unsigned)max_nchunks, (unsigned)tiles);
    cfg.blockDim = dim3(256);
    MFQB_CUDA(cudaLaunchKernelEx(&cfg, x_frag_kernel, fa));
    *xf = frags;
    *down = dn;
}
static void* x16_scratch(int device, size_t bytes, cudaStream_t s) {
    static GrowOnlyScratch pool;
    return pool.get(device, bytes, s, "mfqb_mul_mat (f16 activation fragments)");
}
// y[m, n] = x[m, k] * W^T for 5 <= m <= 16 on the f16 batched kernel
static void launch_bl_gemvh(const NintDevB& w, const void* x, int m, void* y, int y_dtype, int ldy, int device, cudaStream_t s) {
    GemvArgsB a{};
    a.w = w;
    a.y = y;
    a.m = m;
    a.ldy = ldy;
    a.y_dtype = y_dtype;
    const int nt = m > 8 ? 2 : 1, sms = device_sm_count(device);
    XFragArgs fa{};
    fa.x = x;
    fa.k = w.k;
    fa.nt = nt;
    fa.m = m;
    fa.tile_stride = nint_bl_frag_tile_units(w, nt);
    fa.pool_t8[0] = w.t8;
    fa.pool_nchunks[0] = w.nchunks;
    launch_x_frags(fa, m, 1, w.nchunks, x16_scratch(device, x_frags_bytes(m, 1, fa.tile_stride), s), &a.x16f, &a.x16_scale, s);
    a.x16f_tile_stride = fa.tile_stride;
    GemvPlanB p;
    p.passes = nt == 2 ? 116 : 108;
    // at least two row-blocks per CTA where the matrix allows: a chunk's activations then serve several records
    // (tall matrices take several waves of CTAs rather than more than eight row-blocks each)
    const int cap = ctas_per_sm(gemvh_smem(w, 2, nt), 3) * sms;
    p.grid = std::max(1, std::min(w.nrb >= 2 * sms ? w.nrb / 2 : w.nrb, cap));
    a.rb_per_cta = std::min(8, (w.nrb + p.grid - 1) / p.grid);
    p.grid = (w.nrb + a.rb_per_cta - 1) / a.rb_per_cta;
    p.smem = gemvh_smem(w, a.rb_per_cta, nt);
    if (p.smem > kGemvSmemLimit) fail(MFQB_ERR_UNSUPPORTED, "batched product: %d row-blocks per CTA do not fit shared memory", a.rb_per_cta);
    dispatch(a, p, s, "batched GEMV (f16)");
}

// Largest number of two-row passes (4, 2 or 1) whose plane buffers and record rings fit one CTA.
int nint_bl_max_passes(const NintDevB& w) {
    for (int p = 4; p > 1; p /= 2)
        if (gemvn_smem(w, 2, p) <= kGemvSmemLimit) return p;
    return 1;
}

// y[m, n] = x[m, k] * W^T for m <= 8 (the caller loops larger batches).  swiglu (m = 1 only): x is the
// float32 gate|up row [2k] and the product is taken with up * silu(gate).  glu (m = 1 only): the weight's
// 16-row blocks alternate gate and up rows and y [n / 2] receives up * silu(gate).
void launch_bl_gemv(const NintDevB& w, const void* x, int m, void* y, int y_dtype, int ldy, int device, cudaStream_t s, bool swiglu, bool glu) {
    GemvArgsB a{};
    a.w = w;
    a.x = static_cast<const __nv_bfloat16*>(x);
    a.y = y;
    a.m = m;
    a.ldy = ldy;
    a.y_dtype = y_dtype;
    GemvPlanB p;
    const int sms = device_sm_count(device);
    if (m == 1) {
        // three CTAs per SM, all resident at once; row-blocks are split evenly inside the kernel
        const int warps = gemv1_warps(w);
        p.threads = warps * 32;
        p.grid = std::min(w.nrb, ctas_per_sm(gemv1_smem(w, 1, warps), warps > 8 ? 2 : 3) * sms);
        a.rb_per_cta = (w.nrb + p.grid - 1) / p.grid;
        if (glu) {   // (gate, up) pairs of row-blocks stay together
            if ((w.nrb & 1) || (w.n & 31)) fail(MFQB_ERR_ARG, "gated product: the weight needs whole (gate, up) pairs of 16-row blocks, n = %d", w.n);
            p.grid = std::min(w.nrb / 2, p.grid);
            a.rb_per_cta = 2 * ((w.nrb / 2 + p.grid - 1) / p.grid);
            a.glu = 1;
        }
        a.private_sums = gemv1_private_sums(a.rb_per_cta);
        p.smem = gemv1_smem(w, a.rb_per_cta, warps);
        if (swiglu) {
            p.passes = -2;
            a.x_mode = 2;
        }
    } else {
        if (swiglu || glu) fail(MFQB_ERR_ARG, "the fused activation belongs to the single-row kernel");
        if (m >= 5 && m <= 16 && nint_bl_gemvh_supported(w, m)) {   // from five rows on the f16 formulation is cheaper
            launch_bl_gemvh(w, x, m, y, y_dtype, ldy, device, s);
            return;
        }
        const int max_rows = 2 * nint_bl_max_passes(w);
        if (m > max_rows) {   // wide records: the batch goes through in several launches
            const size_t ysz = y_dtype == MFQB_F32 ? 4 : 2;
            for (int m0 = 0; m0 < m; m0 += max_rows)
                launch_bl_gemv(w, static_cast<const char*>(x) + (size_t)m0 * w.k * 2, std::min(max_rows, m - m0),
                               static_cast<char*>(y) + (size_t)m0 * ldy * ysz, y_dtype, ldy, device, s, false, false);
            return;
        }
        launch_x_planes(w, x, m, planes_scratch(device, nint_bl_planes_bytes(w, m), s), &a.xq_g, &a.gtab_g, s, false);
        p.passes = passes_for(m);
        // at least two row-blocks per CTA where the matrix allows: a chunk's planes then serve several items
        const int cap = ctas_per_sm(gemvn_smem(w, 2, p.passes), p.passes == 4 ? 2 : 3) * sms;
        p.grid = std::max(1, std::min(w.nrb >= 2 * sms ? w.nrb / 2 : w.nrb, cap));
        a.rb_per_cta = (w.nrb + p.grid - 1) / p.grid;
        p.smem = gemvn_smem(w, a.rb_per_cta, p.passes);
        if (p.smem > kGemvSmemLimit) fail(MFQB_ERR_UNSUPPORTED, "batched product: %d row-blocks per CTA do not fit shared memory", a.rb_per_cta);
    }
    dispatch(a, p, s, "GEMV");
}

// Single-row product on the residual row with the add + RMSNorm fused in (GemvArgsB::norm_*): y = W . norm(h + delta),
// or the gated form of it (glu).  The normalised row lives in shared memory behind the rings.
void launch_bl_gemv_norm(const NintDevB& w, const float* h, const float* delta, const float* gamma, float eps, float* h_out, void* y, int y_dtype,
                         bool glu, int device, cudaStream_t s) {
    if (w.k % 4) fail(MFQB_ERR_ARG, "fused normalisation needs a row length that is a multiple of 4, got %d", w.k);
    GemvArgsB a{};
    a.w = w;
    a.x = reinterpret_cast<const __nv_bfloat16*>(h);
    a.y = y;
    a.m = 1;
    a.ldy = w.n;
    a.y_dtype = y_dtype;
    a.x_mode = 3;
    a.norm_delta = delta;
    a.norm_gamma = gamma;
    a.norm_eps = eps;
    a.norm_h_out = h_out;
    GemvPlanB p;
    const int warps = gemv1_warps(w), sms = device_sm_count(device);
    const size_t row_bytes = (size_t)w.k * 4;
    p.threads = warps * 32;
    p.passes = -4;
    p.grid = std::min(w.nrb, ctas_per_sm(gemv1_smem(w, 1, warps) + row_bytes, warps > 8 ? 2 : 3) * sms);
    a.rb_per_cta = (w.nrb + p.grid - 1) / p.grid;
    if (glu) {   // (gate, up) pairs of row-blocks stay together
        if ((w.nrb & 1) || (w.n & 31)) fail(MFQB_ERR_ARG, "gated product: the weight needs whole (gate, up) pairs of 16-row blocks, n = %d", w.n);
        p.grid = std::min(w.nrb / 2, p.grid);
        a.rb_per_cta = 2 * ((w.nrb / 2 + p.grid - 1) / p.grid);
        a.glu = 1;
    }
    a.private_sums = gemv1_private_sums(a.rb_per_cta);
    p.smem = gemv1_smem(w, a.rb_per_cta, warps) + row_bytes;
    if (p.smem > kGemvSmemLimit) fail(MFQB_ERR_UNSUPPORTED, "fused normalisation: a row of %d columns does not fit shared memory beside the rings", w.k);
    dispatch(a, p, s, "GEMV with fused RMSNorm");
}

// Streamed single-row product (nint_gemvs.cuh).  `fix` is the weight's own scratch for row-blocks
// that straddle CTAs: [sms][16] (value, flag) pairs, all zero between calls.  Returns false when the
// activation planes of this row length and a useful ring do not fit one CTA; the caller then
// takes the ring kernel.
static cudaError_t dispatch_gemvs(const GemvSArgs& a, const GemvSPlan& p, cudaStream_t s) {
    switch (a.w.bits) {
        case 2: return launch_gemvs_bits<2>(a, p, s);
        case 3: return launch_gemvs_bits<3>(a, p, s);
        case 4: return launch_gemvs_bits<4>(a, p, s);
        case 5: return launch_gemvs_bits<5>(a, p, s);
        case 6: return launch_gemvs_bits<6>(a, p, s);
        case 8: return launch_gemvs_bits<8>(a, p, s);
        default: return cudaErrorInvalidValue;
    }
}

#ifdef MFQB_GEMVS_TRACE
static unsigned long long* g_gemvs_trace = nullptr;
extern "C" __attribute__((visibility("default"))) void mfqb_debug_set_gemvs_trace(void* p) { g_gemvs_trace = static_cast<unsigned long long*>(p); }
#endif

size_t gemvs_fix_bytes(int device) { return (size_t)device_sm_count(device) * 16 * sizeof(uint2); }

bool launch_bl_gemvs(const NintDevB& w, const void* x, int x_dtype, void* y, int y_dtype, int device, void* fix, int* error, cudaStream_t s) {
    if (w.table || !fix || x_dtype != MFQB_BF16) return false;   // lattice records stay on the ring kernel
    const int sms = device_sm_count(device);
    const long long total = (long long)w.nrb * w.nchunks;
    if (total < 1 || total * (sms + 1) >= (1ll << 31)) return false;
    const int grid = (int)std::min<long long>(sms, total);
    const size_t recb = (size_t)w.rec_words * 4;
    const int ngp = w.nchunks * kChunkGroupsB;
    const size_t planes = (size_t)ngp * 16 + 288 + (size_t)ngp * gemvs_group_bytes(w.t8) + 128;   // group table, maxima, sums | zeros | planes
    const long long n_b = (total + grid - 1) / grid;
    GemvSArgs a{};
    GemvSPlan p;
    bool found = false;
    // two CTAs (this product's and the next one's) share an SM when a CTA stays below half of it
    // Most warps first (they hide the latency of the arithmetic and share the staging work), as long as
    // every warp keeps two records in flight.  A CTA below half an SM lets the next product's CTA
    // move in early; records too wide for eight such warps take the whole SM instead.
    struct Try { size_t budget; int warps; };
    for (const Try t : {Try{110 * 1024, 16}, Try{110 * 1024, 12}, Try{110 * 1024, 8}, Try{200 * 1024, 8}, Try{110 * 1024, 4}, Try{200 * 1024, 4}}) {
        const int warps = t.warps;
        if (warps * 32 > gemvs_max_threads(w.wc)) continue;
        const long long n_w = (n_b + warps - 1) / warps;
        const int maxseg = (int)((n_w - 1) / w.nchunks) + 2;
        const int maxrb = (int)(n_b / w.nchunks) + 2;
        const size_t fixed = planes + (size_t)warps * maxseg * 64 + (size_t)(maxrb + 3) / 4 * 16 + 16;
        if (fixed >= t.budget) continue;
        int stages = (int)std::min<size_t>(8, (t.budget - fixed) / (warps * (recb + 8)));
        stages = (int)std::min<long long>(stages, std::max<long long>(n_w, 1));
        const int need = (int)std::min<long long>(2, std::max<long long>(n_w, 1));
        if (stages < need) continue;
        p.grid = grid;
        p.threads = warps * 32;
        p.smem = fixed + (size_t)warps * stages * (recb + 8);
        a.stages = stages;
        a.maxseg = maxseg;
        a.maxrb = maxrb;
        found = true;
        break;
    }
    if (!found) return false;
    a.w = w;
    a.x = x;
    a.x_dtype = x_dtype;
    a.y = y;
    a.y_dtype = y_dtype;
    a.fix_slots = static_cast<uint2*>(fix);
    a.error = error;
#ifdef MFQB_GEMVS_TRACE
    a.trace = g_gemvs_trace;
#endif
    const cudaError_t e = dispatch_gemvs(a, p, s);
    if (e != cudaSuccess) fail(MFQB_ERR_CUDA, "NINT%d gs=%d streamed GEMV launch (%d x %d threads, %zu bytes): %s", w.bits, w.gs, p.grid, p.threads, p.smem,
                               cudaGetErrorString(e));
    return true;
}

// Several weights of one shape class applied to the same activation row in one launch (q|k|v, gate|up:
// the reference's NintLinearGroup, cpp_runtime/mfq_decode.cpp:8618-8743): grid = (CTAs per weight, weights).
void launch_bl_gemv_multi(const NintDevB* ws, void* const* ys, int count, const void* x, int y_dtype, int device, cudaStream_t s) {
    if (count < 1 || count > kGemvMultiMax) fail(MFQB_ERR_ARG, "a multi-weight launch takes 1 to %d weights, got %d", kGemvMultiMax, count);
    GemvArgsB a{};
    a.w = ws[0];
    a.x = static_cast<const __nv_bfloat16*>(x);
    a.m = 1;
    a.y_dtype = y_dtype;
    GemvMultiTable table{};
    int max_nrb = 0;
    for (int i = 0; i < count; ++i) {
        const NintDevB& w = ws[i];
        if (w.table || w.bits != ws[0].bits || w.gs != ws[0].gs || w.k != ws[0].k || w.rec_words != ws[0].rec_words)
            fail(MFQB_ERR_ARG, "the weights of a multi-weight launch must share family, code width, group size and k");
        table.e[i] = GemvMultiEntry{w.items, w.anchors, ys[i], w.n, w.nrb};
        max_nrb = std::max(max_nrb, w.nrb);
    }
    a.ldy = 0;
    GemvPlanB p;
    const int warps = gemv1_warps(ws[0]), sms = device_sm_count(device);
    p.threads = warps * 32;
    p.passes = -1;
    p.multi = &table;
    // all CTAs resident at once: the SMs' slots shared out over the weights
    const int per_weight = std::max(1, ctas_per_sm(gemv1_smem(ws[0], 1, warps), warps > 8 ? 2 : 3) * sms / count);
    a.rb_per_cta = (max_nrb + std::min(max_nrb, per_weight) - 1) / std::min(max_nrb, per_weight);
    p.grid = (max_nrb + a.rb_per_cta - 1) / a.rb_per_cta;   // no more CTAs than that many row-blocks each need: an even split
    p.grid_y = count;
    a.private_sums = gemv1_private_sums(a.rb_per_cta);
    p.smem = gemv1_smem(ws[0], a.rb_per_cta, warps);
    if (p.smem > kGemvSmemLimit) fail(MFQB_ERR_UNSUPPORTED, "multi-weight launch: %d row-blocks per CTA do not fit shared memory", a.rb_per_cta);
    dispatch(a, p, s, "multi-weight GEMV");
}

// Single-row product whose epilogue reduces over ranks (row-parallel shards): see PeerReduce.
void launch_bl_gemv_reduce(const NintDevB& w, const void* x, void* y, int y_dtype, int device, const PeerReduce& pr, cudaStream_t s) {
    GemvArgsB a{};
    a.w = w;
    a.x = static_cast<const __nv_bfloat16*>(x);
    a.y = y;
    a.m = 1;
    a.ldy = w.n;
    a.y_dtype = y_dtype;
    a.reduce = pr;
    GemvPlanB p;
    const int warps = gemv1_warps(w), sms = device_sm_count(device);
    p.threads = warps * 32;
    // Every CTA waits for its peers inside the kernel, so the whole grid must be resident at once: the
    // grid is sized from the occupancy the runtime reports for this kernel, block size and shared memory
    // (which itself grows with the row-blocks per CTA, hence the second look).
    p.grid = std::min(w.nrb, ctas_per_sm(gemv1_smem(w, 1, warps), warps > 8 ? 2 : 3) * sms);
    for (int round = 0; round < 3; ++round) {
        a.rb_per_cta = (w.nrb + p.grid - 1) / p.grid;
        a.private_sums = gemv1_private_sums(a.rb_per_cta);
        p.smem = gemv1_smem(w, a.rb_per_cta, warps);
        if (p.smem > kGemvSmemLimit) fail(MFQB_ERR_UNSUPPORTED, "weight of %d rows is too tall for one resident grid", w.n);
        int per_sm = 0;
        GemvPlanB query = p;
        query.occupancy_out = &per_sm;
        dispatch(a, query, s, "row-parallel GEMV (occupancy)");
        if (per_sm < 1) fail(MFQB_ERR_UNSUPPORTED, "row-parallel GEMV: a CTA of %d threads and %zu bytes does not fit an SM", p.threads, p.smem);
        if (p.grid <= per_sm * sms) break;
        if (round == 2) fail(MFQB_ERR_UNSUPPORTED, "row-parallel GEMV: no grid of this weight's %d row-blocks is resident at once", w.nrb);
        p.grid = per_sm * sms;
    }
    dispatch(a, p, s, "row-parallel GEMV");
}

// Routed single-row launch over (splits, pairs) CTAs for one cohort; see GemvArgsB.
void launch_nint_bl_gemv_routed(GemvArgsB a, int pairs, int device, cudaStream_t s) {
    const NintDevB& w = a.w;
    a.m = 1;
    GemvPlanB p;
    const int want = (3 * device_sm_count(device) + pairs - 1) / std::max(pairs, 1);
    const int splits = std::max(1, std::min(a.rb_per_expert, want));
    a.rb_per_cta = (a.rb_per_expert + splits - 1) / splits;
    a.private_sums = gemv1_private_sums(a.rb_per_cta);
    p.smem = gemv1_smem(w, a.rb_per_cta, 8);
    p.grid = splits;
    p.grid_y = pairs;
    p.passes = -3;
    dispatch(a, p, s, "routed GEMV");
}

// Batched kernel over route-plan tiles (up to tile_m = 2, 4 or 8 pairs of one expert each) for one cohort.
void launch_nint_bl_gemv_tiles(GemvArgsB a, int tile_m, int max_tiles, int device, cudaStream_t s) {
    const NintDevB& w = a.w;
    a.m = tile_m;
    GemvPlanB p;
    p.passes = tile_m / 2;
    // max_tiles is an upper bound and a launch covers one cohort only, so most of its tiles return at
    // once: split an expert's rows finely (about eight row-blocks per CTA) to keep the SMs busy
    const int want = (2 * device_sm_count(device) + max_tiles - 1) / std::max(max_tiles, 1);
    const int splits = std::max(1, std::min(a.rb_per_expert, std::max(a.rb_per_expert / 8, want)));
    a.rb_per_cta = (a.rb_per_expert + splits - 1) / splits;
    p.smem = gemvn_smem(w, a.rb_per_cta, p.passes);
    p.grid = splits;
    p.grid_y = max_tiles;
    dispatch(a, p, s, "routed tile GEMV");
}

}  // namespace mfqb
