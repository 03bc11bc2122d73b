// Dense decoder step around the packed-weight products: the QuantLinear / FFN-shaped runtime layer
// of the reference (cpp_runtime/mfq_decode.cpp:9116-9407 QuantLinear, 10456-10602 FFN,
// 12210-12400 FullBlock::forward, 13993-14145 Model::hidden_forward / next_token) reduced to what one
// decode step of a Llama-shaped model needs: RMSNorm, fused q|k|v projection, rotary embedding, bf16
// KV-cache write, grouped-query decode attention over the cache, output projection, SwiGLU FFN with a
// fused gate|up projection, final norm, lm_head and arg-max.  Every projection is a packed weight
// handle of this library (mfqb_mul_mat); the small kernels here are the glue between them.
//
// Tensor parallelism (Megatron style, as the reference's load_quant_linear assigns axes by tensor
// name, cpp_runtime/mfq_decode.cpp:9422-9443): q/k/v, gate/up and lm_head are split on the output
// axis (heads, FFN columns, vocabulary rows), o_proj and down_proj on the input axis; a rank holds
// n_q/world query heads and n_kv/world KV heads with their slice of the cache.  The two row-parallel
// products of a layer end in a sum over ranks (mfqb_mul_mat_allreduce for one row, product +
// mfqb_allreduce_f32 for a batch), the arg-max over the vocabulary shards in a small gather.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <memory>
#include <vector>

#include <cmath>

#include "cuda_util.h"

namespace mfqb {

constexpr int kHeadDim = 128;

// Every kernel of the step is launched with the programmatic-dependent-launch attribute: it becomes
// resident while its predecessor still runs, and waits here until that one has completed.
__device__ __forceinline__ void dep_wait() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
}
template <typename... KArgs, typename... Args>
static void launch_dep_smem(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t s, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    MFQB_CUDA(cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...));
}
template <typename... KArgs, typename... Args>
static void launch_dep(void (*kernel)(KArgs...), dim3 grid, dim3 block, cudaStream_t s, Args... args) {
    launch_dep_smem(kernel, grid, block, 0, s, args...);
}

// ---- glue kernels --------------------------------------------------------------------------------

// h [rows, H] (float32 residual stream) += delta [rows, H] (optional); xn = h / rms(h) * gamma as bf16.
// One CTA of 1024 threads per row, four columns per thread and pass: a row of up to 8192 columns is
// read once and stays in registers between the sum of squares and the scaling (H is a multiple of 4).
__global__ void __launch_bounds__(1024) add_rmsnorm_kernel(float* __restrict__ h, const float* __restrict__ delta, const float* __restrict__ gamma,
                                                            __nv_bfloat16* __restrict__ xn, int H, float eps) {
    constexpr int KEEP = 2;
    __shared__ float red[32];
    const int tid = threadIdx.x, nv = H >> 2;
    float4* row = reinterpret_cast<float4*>(h + (size_t)blockIdx.x * H);
    const float4* drow = delta ? reinterpret_cast<const float4*>(delta + (size_t)blockIdx.x * H) : nullptr;
    const float4* g4 = reinterpret_cast<const float4*>(gamma);
    uint2* out = reinterpret_cast<uint2*>(xn + (size_t)blockIdx.x * H);
    float4 v[KEEP], g[KEEP];
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
#pragma unroll
    for (int j = 0; j < KEEP; ++j)   // gamma is a constant of the model: fetched while the predecessor still runs
        if (tid + j * 1024 < nv) g[j] = __ldg(g4 + tid + j * 1024);
    asm volatile("griddepcontrol.wait;" ::: "memory");
    float ss = 0.f;
    auto take = [&](int i) {
        float4 t = row[i];
        if (drow) {
            const float4 d = drow[i];
            t.x += d.x; t.y += d.y; t.z += d.z; t.w += d.w;
            row[i] = t;
        }
        ss += t.x * t.x + t.y * t.y + t.z * t.z + t.w * t.w;
        return t;
    };
#pragma unroll
    for (int j = 0; j < KEEP; ++j)
        if (tid + j * 1024 < nv) v[j] = take(tid + j * 1024);
    for (int i = tid + KEEP * 1024; i < nv; i += 1024) take(i);
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if ((tid & 31) == 0) red[tid >> 5] = ss;
    __syncthreads();
    float tot = red[tid & 31];
    for (int o = 16; o > 0; o >>= 1) tot += __shfl_xor_sync(0xffffffffu, tot, o);
    const float inv = rsqrtf(tot / (float)H + eps);
    auto put = [&](int i, const float4& t, const float4& gm) {
        const __nv_bfloat162 lo = __floats2bfloat162_rn(t.x * inv * gm.x, t.y * inv * gm.y), hi = __floats2bfloat162_rn(t.z * inv * gm.z, t.w * inv * gm.w);
        out[i] = make_uint2(*reinterpret_cast<const uint32_t*>(&lo), *reinterpret_cast<const uint32_t*>(&hi));
    };
#pragma unroll
    for (int j = 0; j < KEEP; ++j)
        if (tid + j * 1024 < nv) put(tid + j * 1024, v[j], g[j]);
    for (int i = tid + KEEP * 1024; i < nv; i += 1024) put(i, row[i], __ldg(g4 + i));
}

// cos and sin of position x frequency for the 64 rotation pairs, once per step and sequence:
// table [rows][64] (cos, sin).  The frequencies theta^(-2i/128) come from the host.
__global__ void __launch_bounds__(64) rope_table_kernel(const int* __restrict__ pos, const float* __restrict__ inv_freq, float2* __restrict__ table) {
    dep_wait();
    float sn, cs;
    sincosf((float)pos[blockIdx.x] * inv_freq[threadIdx.x], &sn, &cs);
    table[blockIdx.x * 64 + threadIdx.x] = make_float2(cs, sn);
}

// Rotary embedding (halves convention: pairs (i, i + 64)) of one 128-wide head at `src`: the lane's
// eight dimensions 8 * l16 .. 8 * l16 + 7, times `scale`; tab = the sequence's 64 (cos, sin) pairs.
__device__ __forceinline__ void rope8(const float* __restrict__ src, const float2* __restrict__ tab, int l16, float scale, float* out) {
    const int base = 8 * (l16 & 7);   // pair index i = base + j in [0, 64)
    const float4 lo0 = *reinterpret_cast<const float4*>(src + base), lo1 = *reinterpret_cast<const float4*>(src + base + 4);
    const float4 hi0 = *reinterpret_cast<const float4*>(src + 64 + base), hi1 = *reinterpret_cast<const float4*>(src + 64 + base + 4);
    const float lo[8] = {lo0.x, lo0.y, lo0.z, lo0.w, lo1.x, lo1.y, lo1.z, lo1.w};
    const float hi[8] = {hi0.x, hi0.y, hi0.z, hi0.w, hi1.x, hi1.y, hi1.z, hi1.w};
    const float4* t4 = reinterpret_cast<const float4*>(tab + base);   // two (cos, sin) pairs per load
#pragma unroll
    for (int j = 0; j < 8; j += 2) {
        const float4 t = __ldg(t4 + (j >> 1));
        const float ra0 = lo[j] * t.x - hi[j] * t.y, rb0 = hi[j] * t.x + lo[j] * t.y;
        const float ra1 = lo[j + 1] * t.z - hi[j + 1] * t.w, rb1 = hi[j + 1] * t.z + lo[j + 1] * t.w;
        out[j] = (l16 < 8 ? ra0 : rb0) * scale;
        out[j + 1] = (l16 < 8 ? ra1 : rb1) * scale;
    }
}
__device__ __forceinline__ uint4 pack_bf16x8(const float* f) {
    const __nv_bfloat162 a = __floats2bfloat162_rn(f[0], f[1]), b = __floats2bfloat162_rn(f[2], f[3]);
    const __nv_bfloat162 c = __floats2bfloat162_rn(f[4], f[5]), d = __floats2bfloat162_rn(f[6], f[7]);
    return make_uint4(*reinterpret_cast<const uint32_t*>(&a), *reinterpret_cast<const uint32_t*>(&b), *reinterpret_cast<const uint32_t*>(&c),
                      *reinterpret_cast<const uint32_t*>(&d));
}
__device__ __forceinline__ void bf16x8_to_f32(const uint4& r, float* f) {
    f[0] = __uint_as_float(r.x << 16); f[1] = __uint_as_float(r.x & 0xFFFF0000u);
    f[2] = __uint_as_float(r.y << 16); f[3] = __uint_as_float(r.y & 0xFFFF0000u);
    f[4] = __uint_as_float(r.z << 16); f[5] = __uint_as_float(r.z & 0xFFFF0000u);
    f[6] = __uint_as_float(r.w << 16); f[7] = __uint_as_float(r.w & 0xFFFF0000u);
}

constexpr int kMaxSplits = 64;
constexpr int kAttnStages = 3;   // rounds of 32 tokens in flight per CTA
// Dynamic shared memory of the attention kernel: the K/V ring (stages x 4 tokens x (K, V) x 128 threads x 16 bytes),
// reused afterwards for the eight half-warps' results ([8][G][128] + 2 x [8][G] floats).
constexpr size_t attn_smem_bytes(int g) {
    const size_t ring = (size_t)kAttnStages * 4 * 2 * 128 * 16, meet = (size_t)8 * g * (kHeadDim + 2) * 4;
    return ring > meet ? ring : meet;
}
__device__ __forceinline__ void cp_async16_attn(void* smem_dst, const void* gsrc) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"((uint32_t)__cvta_generic_to_shared(smem_dst)), "l"(gsrc) : "memory");
}
constexpr int kPartStride = kHeadDim + 4;   // a split's record per head: 128 output values | max | sum | pad (528 bytes)

// Grouped-query decode attention for one new token per sequence, one launch: rotary embedding,
// cache write, scan and merge.  qkv [rows, (nq + 2 nkv) * 128] float32 is the fused projection;
// the caches are [rows][nkv][max_ctx][128] bf16 for K and for V.
//
// CTA (split, kv head, row) scans its slice of the context for the G = nq / nkv query heads that share
// the KV head.  Every CTA rotates those heads' queries itself (pre-scaled by 1/sqrt(128)); the CTA
// whose slice holds the new position rotates the new key, rounds key and value to bf16 and writes
// them into the caches before it scans (no other CTA reads that position in this step).  A
// half-warp holds one token (16 lanes x 8 dimensions = one 16-byte load per lane for K and for V);
// the CTA's eight half-warps take four tokens each per round of 32, eight 16-byte loads per lane in
// flight, the first round requested before the queries are rotated.  Scores are reduced inside the
// half-warp, the soft-max runs online per half-warp and head.  Each CTA leaves (unnormalised
// output[128], max, sum) per head in `part`; the last CTA of a (row, kv head) to arrive -- a counter
// per pair, left at zero -- merges the splits, a warp per head, and writes the bf16 attention output.
template <int G>
__global__ void __launch_bounds__(128, G <= 4 ? 4 : 2) attn_decode_kernel(const float* __restrict__ qkv, __nv_bfloat16* kcache, __nv_bfloat16* vcache,
                                                             const int* __restrict__ pos, float* part, unsigned* counters,
                                                             __nv_bfloat16* __restrict__ out, int nq, int nkv, int max_ctx, int nsplit,
                                                             const float2* __restrict__ rope_table) {
    dep_wait();
    const int split = blockIdx.x, kvh = blockIdx.y, row = blockIdx.z;
    const int lane = threadIdx.x & 31, l16 = lane & 15, slot = threadIdx.x >> 4;   // slot: half-warp 0..7 of the CTA
    const int p = pos[row], len = p + 1;   // the token written by this step takes part
    const int per = (len + nsplit - 1) / nsplit;
    const int t0 = split * per, t1 = min(len, t0 + per);
    const float* qkv_row = qkv + (size_t)row * (nq + 2 * nkv) * kHeadDim;
    const float2* tab = rope_table + (size_t)row * 64;
    __nv_bfloat16* kb = kcache + ((size_t)row * nkv + kvh) * max_ctx * kHeadDim + 8 * l16;
    __nv_bfloat16* vb = vcache + ((size_t)row * nkv + kvh) * max_ctx * kHeadDim + 8 * l16;
    if (t0 <= p && p < t1) {   // this CTA's slice holds the new position (uniform over the CTA)
        if (threadIdx.x < 32) {   // warp 0 writes the new key and value
            float f[8];
            if (lane < 16) {
                rope8(qkv_row + (size_t)(nq + kvh) * kHeadDim, tab, l16, 1.0f, f);
                *reinterpret_cast<uint4*>(kb + (size_t)p * kHeadDim) = pack_bf16x8(f);
            } else {
                const float* src = qkv_row + (size_t)(nq + nkv + kvh) * kHeadDim + 8 * l16;
                const float4 a = *reinterpret_cast<const float4*>(src), b = *reinterpret_cast<const float4*>(src + 4);
                f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
                *reinterpret_cast<uint4*>(vb + (size_t)p * kHeadDim) = pack_bf16x8(f);
            }
        }
        __syncthreads();   // visible to the whole CTA before anyone reads that position
    }
    // A half-warp takes four tokens per round (slot, slot + 8, + 16, + 24 of a 32-token round).  Every lane copies
    // the 16 bytes of K and of V it will use itself into its own slots of a ring in shared memory, kAttnStages
    // rounds deep (asynchronous copies, no registers held, no synchronisation: a lane only reads what it copied),
    // so the loads of the next rounds are in flight while a round is used.
    constexpr int TPR = 4;
    extern __shared__ __align__(16) unsigned char attn_smem[];
    uint4* ring = reinterpret_cast<uint4*>(attn_smem);   // [stage][token of the round][K, V][thread]
    auto slot_of = [&](int stage, int i, int kv) { return ring + ((stage * TPR + i) * 2 + kv) * 128 + threadIdx.x; };
    auto request = [&](int base, int stage) {   // one copy group per round, empty past the end of the slice
#pragma unroll
        for (int i = 0; i < TPR; ++i) {
            const int t = base + slot + 8 * i;
            if (t < t1) {
                cp_async16_attn(slot_of(stage, i, 0), kb + (size_t)t * kHeadDim);
                cp_async16_attn(slot_of(stage, i, 1), vb + (size_t)t * kHeadDim);
            }
        }
        asm volatile("cp.async.commit_group;\n" ::: "memory");
    };
#pragma unroll
    for (int sidx = 0; sidx < kAttnStages - 1; ++sidx) request(t0 + sidx * 8 * TPR, sidx);
    float qv[G][8];
    if (t0 < t1) {
#pragma unroll
        for (int g = 0; g < G; ++g) rope8(qkv_row + (size_t)(kvh * G + g) * kHeadDim, tab, l16, 0.08838834764831845f /* 1/sqrt(128) */, qv[g]);
    }
    float m[G], l[G], acc[G][8];
#pragma unroll
    for (int g = 0; g < G; ++g) {
        m[g] = -INFINITY;
        l[g] = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[g][i] = 0.f;
    }
    const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
    int stage = 0, req_stage = kAttnStages - 1;
    for (int base = t0; base < t1; base += 8 * TPR) {   // uniform trip count over the CTA: the shuffles below need whole warps
        request(base + (kAttnStages - 1) * 8 * TPR, req_stage);   // the slot read in the previous iteration
        asm volatile("cp.async.wait_group %0;\n" ::"n"(kAttnStages - 1) : "memory");
        float sc[TPR][G];
#pragma unroll
        for (int i = 0; i < TPR; ++i) {
            float kf[8];
            const uint4 ck = base + slot + 8 * i < t1 ? *slot_of(stage, i, 0) : zero;
            bf16x8_to_f32(ck, kf);
#pragma unroll
            for (int g = 0; g < G; ++g) {
                float x = 0.f;
#pragma unroll
                for (int d = 0; d < 8; ++d) x += qv[g][d] * kf[d];
                sc[i][g] = x;
            }
        }
#pragma unroll
        for (int o = 8; o > 0; o >>= 1)
#pragma unroll
            for (int i = 0; i < TPR; ++i)
#pragma unroll
                for (int g = 0; g < G; ++g) sc[i][g] += __shfl_xor_sync(0xffffffffu, sc[i][g], o);
        if (base + slot < t1) {   // uniform over the half-warp; a later token of the round is valid only if the earlier ones are
            float pr[TPR][G];
#pragma unroll
            for (int g = 0; g < G; ++g) {
                float mn = m[g];
#pragma unroll
                for (int i = 0; i < TPR; ++i) {
                    if (base + slot + 8 * i >= t1) sc[i][g] = -INFINITY;
                    mn = fmaxf(mn, sc[i][g]);
                }
                const float corr = __expf(m[g] - mn);
                float ps = 0.f;
#pragma unroll
                for (int i = 0; i < TPR; ++i) {
                    pr[i][g] = __expf(sc[i][g] - mn);
                    ps += pr[i][g];
                }
                l[g] = l[g] * corr + ps;
#pragma unroll
                for (int d = 0; d < 8; ++d) acc[g][d] *= corr;
                m[g] = mn;
            }
#pragma unroll
            for (int i = 0; i < TPR; ++i) {
                float vf[8];
                const uint4 cv = base + slot + 8 * i < t1 ? *slot_of(stage, i, 1) : zero;
                bf16x8_to_f32(cv, vf);
#pragma unroll
                for (int g = 0; g < G; ++g)
#pragma unroll
                    for (int d = 0; d < 8; ++d) acc[g][d] += pr[i][g] * vf[d];
            }
        }
        if (++stage == kAttnStages) stage = 0;
        if (++req_stage == kAttnStages) req_stage = 0;
    }
    asm volatile("cp.async.wait_group 0;\n" ::: "memory");
    __syncthreads();   // the ring is done with: its memory now holds the half-warps' results
    // the eight half-warps of the CTA meet in shared memory
    float(*sm_acc)[G][kHeadDim] = reinterpret_cast<float(*)[G][kHeadDim]>(attn_smem);                       // [8][G][128]
    float(*sm_m)[G] = reinterpret_cast<float(*)[G]>(attn_smem + (size_t)8 * G * kHeadDim * 4);              // [8][G]
    float(*sm_l)[G] = reinterpret_cast<float(*)[G]>(attn_smem + (size_t)8 * G * kHeadDim * 4 + 8 * G * 4);  // [8][G]
#pragma unroll
    for (int g = 0; g < G; ++g) {
        if (l16 == 0) { sm_m[slot][g] = m[g]; sm_l[slot][g] = l[g]; }
        float4* dst = reinterpret_cast<float4*>(&sm_acc[slot][g][8 * l16]);
        dst[0] = make_float4(acc[g][0], acc[g][1], acc[g][2], acc[g][3]);
        dst[1] = make_float4(acc[g][4], acc[g][5], acc[g][6], acc[g][7]);
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < G * kHeadDim; idx += blockDim.x) {
        const int g = idx / kHeadDim, d = idx % kHeadDim;
        float mm = -INFINITY;
#pragma unroll
        for (int w = 0; w < 8; ++w) mm = fmaxf(mm, sm_m[w][g]);
        float ll = 0.f, aa = 0.f;
#pragma unroll
        for (int w = 0; w < 8; ++w) {
            const float c = sm_m[w][g] == -INFINITY ? 0.f : __expf(sm_m[w][g] - mm);
            ll += sm_l[w][g] * c;
            aa += sm_acc[w][g][d] * c;
        }
        float* dst = part + (((size_t)row * nq + kvh * G + g) * nsplit + split) * kPartStride;
        dst[d] = aa;
        if (d == 0) { dst[kHeadDim] = mm; dst[kHeadDim + 1] = ll; }
    }
    // the last CTA of this (row, kv head) merges the splits: a warp per head, a lane per four dimensions
    __shared__ unsigned s_prev;
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) s_prev = atomicAdd(counters + (size_t)row * nkv + kvh, 1u);
    __syncthreads();
    if (s_prev != (unsigned)(nsplit - 1)) return;
    __threadfence();
    for (int g = threadIdx.x >> 5; g < G; g += 4) {
        const float* src = part + ((size_t)row * nq + kvh * G + g) * nsplit * kPartStride;
        // weights of the splits (nsplit <= 64: two per lane)
        const bool h0 = lane < nsplit, h1 = lane + 32 < nsplit;
        const float2 ml0 = h0 ? __ldcg(reinterpret_cast<const float2*>(src + (size_t)lane * kPartStride + kHeadDim)) : make_float2(-INFINITY, 0.f);
        const float2 ml1 = h1 ? __ldcg(reinterpret_cast<const float2*>(src + (size_t)(lane + 32) * kPartStride + kHeadDim)) : make_float2(-INFINITY, 0.f);
        float mm = fmaxf(ml0.x, ml1.x);
        for (int o = 16; o > 0; o >>= 1) mm = fmaxf(mm, __shfl_xor_sync(0xffffffffu, mm, o));
        const float c0 = ml0.x == -INFINITY ? 0.f : __expf(ml0.x - mm), c1 = ml1.x == -INFINITY ? 0.f : __expf(ml1.x - mm);
        float ll = ml0.y * c0 + ml1.y * c1;
        for (int o = 16; o > 0; o >>= 1) ll += __shfl_xor_sync(0xffffffffu, ll, o);
        float4 aa = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 16
        for (int sp = 0; sp < nsplit; ++sp) {
            const float c = __shfl_sync(0xffffffffu, sp < 32 ? c0 : c1, sp & 31);
            const float4 v = __ldcg(reinterpret_cast<const float4*>(src + (size_t)sp * kPartStride) + lane);
            aa.x += c * v.x; aa.y += c * v.y; aa.z += c * v.z; aa.w += c * v.w;
        }
        const float inv = 1.0f / ll;
        const __nv_bfloat162 o01 = __floats2bfloat162_rn(aa.x * inv, aa.y * inv), o23 = __floats2bfloat162_rn(aa.z * inv, aa.w * inv);
        *reinterpret_cast<uint2*>(out + ((size_t)row * nq + kvh * G + g) * kHeadDim + 4 * lane) =
            make_uint2(*reinterpret_cast<const uint32_t*>(&o01), *reinterpret_cast<const uint32_t*>(&o23));
    }
    if (threadIdx.x == 0) counters[(size_t)row * nkv + kvh] = 0u;
}

// logits [rows, n] float32 -> (largest value, its index + index_base) per row; ties go to the smaller index.
// Two launches: kArgmaxSlices CTAs per row take the best of a slice each, one warp per row merges them.
constexpr int kArgmaxSlices = 64;
__device__ __forceinline__ void argmax_take(float v, int i, float& bv, int& bi) {
    if (v > bv || (v == bv && i < bi)) { bv = v; bi = i; }
}
__global__ void __launch_bounds__(256) argmax_slices_kernel(const float* __restrict__ logits, int n, float* __restrict__ part_val, int* __restrict__ part_idx) {
    dep_wait();
    __shared__ float sv[8];
    __shared__ int si[8];
    const float* row = logits + (size_t)blockIdx.y * n;
    const int per = (n + kArgmaxSlices - 1) / kArgmaxSlices, i0 = blockIdx.x * per, i1 = min(n, i0 + per);
    float bv = -INFINITY;
    int bi = 0x7FFFFFFF;
#pragma unroll 4
    for (int i = i0 + threadIdx.x; i < i1; i += 256) argmax_take(row[i], i, bv, bi);
    for (int o = 16; o > 0; o >>= 1) argmax_take(__shfl_xor_sync(0xffffffffu, bv, o), __shfl_xor_sync(0xffffffffu, bi, o), bv, bi);
    if ((threadIdx.x & 31) == 0) { sv[threadIdx.x >> 5] = bv; si[threadIdx.x >> 5] = bi; }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < 8; ++w) argmax_take(sv[w], si[w], bv, bi);
        part_val[blockIdx.y * kArgmaxSlices + blockIdx.x] = bv;
        part_idx[blockIdx.y * kArgmaxSlices + blockIdx.x] = bi;
    }
}
__global__ void __launch_bounds__(32) argmax_merge_kernel(const float* __restrict__ part_val, const int* __restrict__ part_idx, int index_base,
                                                          float* __restrict__ best_val, int* __restrict__ best_idx) {
    dep_wait();
    const int lane = threadIdx.x;
    float bv = -INFINITY;
    int bi = 0x7FFFFFFF;
    for (int j = lane; j < kArgmaxSlices; j += 32) argmax_take(part_val[blockIdx.x * kArgmaxSlices + j], part_idx[blockIdx.x * kArgmaxSlices + j], bv, bi);
    for (int o = 16; o > 0; o >>= 1) argmax_take(__shfl_xor_sync(0xffffffffu, bv, o), __shfl_xor_sync(0xffffffffu, bi, o), bv, bi);
    if (lane == 0) { best_val[blockIdx.x] = bv; best_idx[blockIdx.x] = bi + index_base; }
}

// Vocabulary shards: gathered [world][rows] (value, index as float) -> winning token per row (smaller rank on ties).
__global__ void argmax_pick_kernel(const float* __restrict__ gathered, int world, int rows, int* __restrict__ token) {
    dep_wait();
    const int r = blockIdx.x * blockDim.x + threadIdx.x;
    if (r >= rows) return;
    float bv = -INFINITY;
    int bi = 0;
    for (int w = 0; w < world; ++w) {
        const float v = gathered[((size_t)w * rows + r) * 2], idx = gathered[((size_t)w * rows + r) * 2 + 1];
        if (v > bv) { bv = v; bi = (int)idx; }
    }
    token[r] = bi;
}
// This rank's (value, index) pairs into its slot of a zeroed [world][rows][2] vector (summing the ranks' vectors gathers them).
__global__ void argmax_pack_kernel(const float* __restrict__ val, const int* __restrict__ idx, int rank, int world, int rows, float* __restrict__ out) {
    dep_wait();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= world * rows * 2) return;
    const int w = i / (rows * 2), r = (i / 2) % rows, f = i & 1;
    out[i] = w == rank ? (f ? (float)idx[r] : val[r]) : 0.f;
}

// Embedding rows: h[r, :] = table[ids[r], :] (bf16 table) as float32.
__global__ void embed_rows_kernel(const int* __restrict__ ids, const __nv_bfloat16* __restrict__ table, float* __restrict__ h, int H, int vocab) {
    dep_wait();
    const int r = blockIdx.x;
    const int id = min(max(ids[r], 0), vocab - 1);
    const uint2* src = reinterpret_cast<const uint2*>(table + (size_t)id * H);   // H is a multiple of 8: four bf16 per load
    float4* dst = reinterpret_cast<float4*>(h + (size_t)r * H);
    for (int i = threadIdx.x; i < (H >> 2); i += blockDim.x) {
        const uint2 v = __ldg(src + i);
        dst[i] = make_float4(__uint_as_float(v.x << 16), __uint_as_float(v.x & 0xFFFF0000u), __uint_as_float(v.y << 16), __uint_as_float(v.y & 0xFFFF0000u));
    }
}

// Seeded synthetic cache contents (a stand-in for the prefill pass): values of unit scale.
__global__ void fill_cache_kernel(__nv_bfloat16* __restrict__ p, size_t n, unsigned seed) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        unsigned x = (unsigned)i * 2654435761u ^ seed ^ (unsigned)(i >> 32) * 40503u;
        x ^= x >> 16; x *= 0x7feb352du; x ^= x >> 15; x *= 0x846ca68bu; x ^= x >> 16;
        p[i] = __float2bfloat16_rn(((float)(x & 0xFFFF) - 32768.f) * (1.f / 18918.f));   // uniform, unit variance
    }
}
__global__ void fill_f32_kernel(float* p, size_t n, float v) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) p[i] = v;
}
__global__ void add_one_kernel(int* p, int n) {
    dep_wait();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) p[i] += 1;
}

}  // namespace mfqb

using namespace mfqb;

struct DecoderLayer {
    const mfqb_weight *qkv = nullptr, *o = nullptr, *gate_up = nullptr, *down = nullptr;   // borrowed handles
    DevBuf gamma_attn, gamma_ffn;                                                        // [H] float32
    DevBuf kcache, vcache;                                                               // [batch][nkv_local][max_ctx][128] bf16
};

struct mfqb_decoder {
    mfqb_decoder_config cfg{};
    int rank = 0, world = 1, device = 0;
    mfqb_comm* comm = nullptr;       // borrowed; null when world == 1
    int nq = 0, nkv = 0, f = 0, vshard = 0, vbase = 0, sms = 0, attn_per_sm = 4;
    // Single-row steps could run the residual add + RMSNorm inside the q|k|v, gate|up and lm_head products
    // (mfqb_mul_mat_rmsnorm).  Measured on the 8B-shaped model it loses: every CTA of those products repeats the
    // normalisation of the row (2.29 against 2.14 ms per step), so the two-kernel form stays the default.
    bool fused_norm = false;
    std::vector<DecoderLayer> layers;
    const mfqb_weight* lm_head = nullptr;
    const void* embedding = nullptr;   // bf16 [vocab, H] on the device, borrowed
    DevBuf gamma_final;
    // workspaces
    DevBuf h, h2, xn, qkv, attn, attn_count, inv_freq, rope_table, proj, proj_sum, act, logits, part, best_val, best_idx, part_val, part_idx, gathered, gathered_sum, pos;
};

// Context splits of the decode attention: as many CTAs as are resident at once (one wave: the merge
// by the last CTA of a head group then follows the scan directly), but at least so many that a CTA
// scans no more than 256 positions of a long context.
static int attn_splits(const mfqb_decoder* d, int rows, int ctx_bound) {
    const int one_wave = d->attn_per_sm * d->sms / (d->nkv * rows);
    const int by_length = (ctx_bound + 255) / 256;
    return std::max(1, std::min(kMaxSplits, std::max(one_wave, by_length)));
}

// The step's rotation table (cos, sin per sequence and pair), before the first block that uses it.
static void launch_rope_table(mfqb_decoder* d, int rows, cudaStream_t s) {
    launch_dep(rope_table_kernel, dim3(rows), dim3(64), s, static_cast<const int*>(d->pos.p), static_cast<const float*>(d->inv_freq.p),
               static_cast<float2*>(d->rope_table.p));
}

static void check_weight_shape(const mfqb_weight* w, int64_t n, int64_t k, const char* what) {
    mfqb_weight_info info;
    if (mfqb_weight_info_get(w, &info) != MFQB_OK) fail(MFQB_ERR_ARG, "%s: bad weight handle", what);
    if (info.n != n || info.k != k) fail(MFQB_ERR_ARG, "%s must be [%lld, %lld], got [%lld, %lld]", what, (long long)n, (long long)k, (long long)info.n, (long long)info.k);
}

static void launch_fill_f32(void* p, size_t n, float v, cudaStream_t s) {
    fill_f32_kernel<<<(unsigned)std::min<size_t>((n + 255) / 256, 1024), 256, 0, s>>>(static_cast<float*>(p), n, v);
}

// sum over ranks of a float32 vector (in place semantics: out may equal in is not allowed by the collective, hence two buffers)
static const float* rank_sum(mfqb_decoder* d, const float* in, float* out, size_t n, cudaStream_t s) {
    if (d->world == 1) return in;
    const int rc = mfqb_allreduce_f32(d->comm, in, out, n, s);
    if (rc != MFQB_OK) throw Error(rc, mfqb_last_error());
    return out;
}

static void mul_mat(const mfqb_weight* w, const void* x, int m, void* y, cudaStream_t s) {
    const int rc = mfqb_mul_mat(w, x, m, y, MFQB_F32, s);
    if (rc != MFQB_OK) throw Error(rc, mfqb_last_error());
}

// One transformer block on the residual stream d->h for `rows` sequences; `delta` is the previous
// block's (already rank-summed) FFN output still to be added, and on return `*delta_out` is this
// block's: the add is fused into the next RMSNorm.
static const float* layer_forward(mfqb_decoder* d, int li, int rows, const float* delta, cudaStream_t s) {
    DecoderLayer& L = d->layers[li];
    const int H = d->cfg.hidden;
    const int G = d->cfg.n_q_heads / d->cfg.n_kv_heads;
    // One row: the residual add and the normalisation run inside the products that consume them (h + delta goes to
    // h2, h2 + attention output back to h).  Batches: a normalisation kernel, then the batched product.
    bool fused = rows == 1 && d->fused_norm;
    if (fused) {
        const int rc = mfqb_mul_mat_rmsnorm(L.qkv, static_cast<const float*>(d->h.p), delta, static_cast<const float*>(L.gamma_attn.p), d->cfg.rms_eps,
                                            static_cast<float*>(d->h2.p), d->qkv.p, MFQB_F32, 0, s);
        if (rc == MFQB_ERR_UNSUPPORTED) d->fused_norm = fused = false;   // weights this form does not take: the two-kernel form from here on
        else if (rc != MFQB_OK) throw Error(rc, mfqb_last_error());
    }
    if (!fused) {
        launch_dep(add_rmsnorm_kernel, dim3(rows), dim3(1024), s, static_cast<float*>(d->h.p), delta, static_cast<const float*>(L.gamma_attn.p),
                   static_cast<__nv_bfloat16*>(d->xn.p), H, d->cfg.rms_eps);
        mul_mat(L.qkv, d->xn.p, rows, d->qkv.p, s);
    }
    const int nsplit = attn_splits(d, rows, d->cfg.max_ctx);
    const dim3 agrid(nsplit, d->nkv, rows);
    auto attn = [&](auto kernel) {
        launch_dep_smem(kernel, agrid, dim3(128), attn_smem_bytes(G), s, static_cast<const float*>(d->qkv.p), static_cast<__nv_bfloat16*>(L.kcache.p),
                   static_cast<__nv_bfloat16*>(L.vcache.p), static_cast<const int*>(d->pos.p), static_cast<float*>(d->part.p),
                   static_cast<unsigned*>(d->attn_count.p), static_cast<__nv_bfloat16*>(d->attn.p), d->nq, d->nkv, d->cfg.max_ctx, nsplit,
                   static_cast<const float2*>(d->rope_table.p));
    };
    switch (G) {
        case 1: attn(attn_decode_kernel<1>); break;
        case 2: attn(attn_decode_kernel<2>); break;
        case 4: attn(attn_decode_kernel<4>); break;
        case 8: attn(attn_decode_kernel<8>); break;
        default: fail(MFQB_ERR_UNSUPPORTED, "query heads per KV head must be 1, 2, 4 or 8, got %d", G);
    }
    // output projection: row-parallel under tensor parallelism
    const float* o_out;
    if (d->world > 1 && rows == 1) {
        const int rc = mfqb_mul_mat_allreduce(L.o, d->attn.p, 1, d->comm, d->proj_sum.p, MFQB_F32, s);
        if (rc != MFQB_OK) throw Error(rc, mfqb_last_error());
        o_out = static_cast<const float*>(d->proj_sum.p);
    } else {
        mul_mat(L.o, d->attn.p, rows, d->proj.p, s);
        o_out = rank_sum(d, static_cast<const float*>(d->proj.p), static_cast<float*>(d->proj_sum.p), (size_t)rows * H, s);
    }
    // gate|up with the activation in the epilogue: the fused weight alternates 16-row blocks of gate and up rows
    if (fused) {
        const int rc = mfqb_mul_mat_rmsnorm(L.gate_up, static_cast<const float*>(d->h2.p), o_out, static_cast<const float*>(L.gamma_ffn.p), d->cfg.rms_eps,
                                            static_cast<float*>(d->h.p), d->act.p, MFQB_BF16, 1, s);
        if (rc != MFQB_OK) throw Error(rc, mfqb_last_error());
    } else {
        launch_dep(add_rmsnorm_kernel, dim3(rows), dim3(1024), s, static_cast<float*>(d->h.p), o_out, static_cast<const float*>(L.gamma_ffn.p),
                   static_cast<__nv_bfloat16*>(d->xn.p), H, d->cfg.rms_eps);
        const int rc = mfqb_mul_mat_glu(L.gate_up, d->xn.p, rows, d->act.p, MFQB_BF16, s);
        if (rc != MFQB_OK) throw Error(rc, mfqb_last_error());
    }
    if (d->world > 1 && rows == 1) {
        const int rc = mfqb_mul_mat_allreduce(L.down, d->act.p, 1, d->comm, d->proj_sum.p, MFQB_F32, s);
        if (rc != MFQB_OK) throw Error(rc, mfqb_last_error());
        return static_cast<const float*>(d->proj_sum.p);
    }
    mul_mat(L.down, d->act.p, rows, d->proj.p, s);
    return rank_sum(d, static_cast<const float*>(d->proj.p), static_cast<float*>(d->proj_sum.p), (size_t)rows * H, s);
}

extern "C" {
#pragma GCC visibility push(default)

int mfqb_decoder_create(const mfqb_decoder_config* cfg, int rank, int world, mfqb_comm* comm, int device, mfqb_decoder** out) {
    return guarded([&] {
        if (!cfg || !out) fail(MFQB_ERR_ARG, "mfqb_decoder_create: null argument");
        if (world < 1 || rank < 0 || rank >= world) fail(MFQB_ERR_ARG, "mfqb_decoder_create: rank %d / world %d", rank, world);
        if (world > 1 && !comm) fail(MFQB_ERR_ARG, "mfqb_decoder_create: tensor parallelism needs a communicator");
        if (cfg->head_dim != kHeadDim) fail(MFQB_ERR_UNSUPPORTED, "head_dim must be %d", kHeadDim);
        if (cfg->n_q_heads % cfg->n_kv_heads || cfg->n_kv_heads % world || cfg->ffn % world || cfg->layers < 1 || cfg->max_batch < 1 ||
            cfg->hidden != cfg->n_q_heads * kHeadDim || cfg->hidden % 8 || (cfg->ffn / world) % 16)
            fail(MFQB_ERR_ARG, "mfqb_decoder_create: head counts, FFN width and hidden size must divide over %d ranks (hidden = heads x 128)", world);
        auto d = std::make_unique<mfqb_decoder>();
        d->cfg = *cfg;
        d->rank = rank;
        d->world = world;
        d->comm = world > 1 ? comm : nullptr;
        d->device = device;
        d->sms = device_sm_count(device);
        d->nq = cfg->n_q_heads / world;
        d->nkv = cfg->n_kv_heads / world;
        d->f = cfg->ffn / world;
        // vocabulary rows in shards of whole 16-row blocks
        const int per = ((cfg->vocab + world - 1) / world + 15) / 16 * 16;
        d->vbase = std::min(cfg->vocab, rank * per);
        d->vshard = std::max(0, std::min(cfg->vocab, d->vbase + per) - d->vbase);
        DeviceGuard guard(device);
        const size_t B = cfg->max_batch, H = cfg->hidden;
        d->layers.resize(cfg->layers);
        for (auto& L : d->layers) {
            L.gamma_attn.alloc(H * 4);
            L.gamma_ffn.alloc(H * 4);
            launch_fill_f32(L.gamma_attn.p, H, 1.f, nullptr);
            launch_fill_f32(L.gamma_ffn.p, H, 1.f, nullptr);
            const size_t cache = B * d->nkv * cfg->max_ctx * kHeadDim * 2;
            L.kcache.alloc(cache);
            L.vcache.alloc(cache);
        }
        d->gamma_final.alloc(H * 4);
        launch_fill_f32(d->gamma_final.p, H, 1.f, nullptr);
        d->h.alloc(B * H * 4);
        d->h2.alloc(B * H * 4);
        d->xn.alloc(B * H * 2);
        d->qkv.alloc(B * (d->nq + 2 * d->nkv) * kHeadDim * 4);
        {   // rotary frequencies theta^(-2i/128), i = 0..63
            float freq[kHeadDim / 2];
            for (int i = 0; i < kHeadDim / 2; ++i) freq[i] = (float)std::pow((double)cfg->rope_theta, -2.0 * i / kHeadDim);
            d->inv_freq.alloc(sizeof(freq));
            MFQB_CUDA(cudaMemcpy(d->inv_freq.p, freq, sizeof(freq), cudaMemcpyHostToDevice));
        }
        {   // resident CTAs per SM of the attention kernel this model uses
            int per_sm = 0;
            cudaError_t e = cudaErrorInvalidValue;
            switch (cfg->n_q_heads / cfg->n_kv_heads) {
                case 1:
                    MFQB_CUDA(cudaFuncSetAttribute(attn_decode_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)attn_smem_bytes(1)));
                    e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, attn_decode_kernel<1>, 128, attn_smem_bytes(1));
                    break;
                case 2:
                    MFQB_CUDA(cudaFuncSetAttribute(attn_decode_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)attn_smem_bytes(2)));
                    e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, attn_decode_kernel<2>, 128, attn_smem_bytes(2));
                    break;
                case 4:
                    MFQB_CUDA(cudaFuncSetAttribute(attn_decode_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)attn_smem_bytes(4)));
                    e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, attn_decode_kernel<4>, 128, attn_smem_bytes(4));
                    break;
                case 8:
                    MFQB_CUDA(cudaFuncSetAttribute(attn_decode_kernel<8>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)attn_smem_bytes(8)));
                    e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, attn_decode_kernel<8>, 128, attn_smem_bytes(8));
                    break;
                default: fail(MFQB_ERR_UNSUPPORTED, "query heads per KV head must be 1, 2, 4 or 8, got %d", cfg->n_q_heads / cfg->n_kv_heads);
            }
            MFQB_CUDA(e);
            d->attn_per_sm = std::max(1, per_sm);
        }
        d->attn_count.alloc(B * d->nkv * 4);
        MFQB_CUDA(cudaMemset(d->attn_count.p, 0, B * d->nkv * 4));
        d->attn.alloc(B * d->nq * kHeadDim * 2);
        d->proj.alloc(B * H * 4);
        d->proj_sum.alloc(B * H * 4);
        d->act.alloc(B * d->f * 2);
        d->logits.alloc(B * std::max(d->vshard, 1) * 4);
        d->part.alloc(B * d->nq * kMaxSplits * kPartStride * 4);
        d->rope_table.alloc(B * 64 * sizeof(float2));
        d->best_val.alloc(B * 4);
        d->part_val.alloc(B * kArgmaxSlices * 4);
        d->part_idx.alloc(B * kArgmaxSlices * 4);
        d->best_idx.alloc(B * 4);
        d->gathered.alloc((size_t)world * B * 2 * 4);
        d->gathered_sum.alloc((size_t)world * B * 2 * 4);
        d->pos.alloc(B * 4);
        MFQB_CUDA(cudaMemset(d->pos.p, 0, B * 4));
        MFQB_CUDA(cudaDeviceSynchronize());
        *out = d.release();
    });
}

int mfqb_decoder_set_layer(mfqb_decoder* d, int layer, const mfqb_weight* qkv, const mfqb_weight* o, const mfqb_weight* gate_up,
                           const mfqb_weight* down) {
    return guarded([&] {
        if (!d || !qkv || !o || !gate_up || !down || layer < 0 || layer >= d->cfg.layers) fail(MFQB_ERR_ARG, "mfqb_decoder_set_layer: bad argument");
        const int64_t H = d->cfg.hidden;
        check_weight_shape(qkv, (int64_t)(d->nq + 2 * d->nkv) * kHeadDim, H, "qkv (query | key | value rows of this rank)");
        check_weight_shape(o, H, (int64_t)d->nq * kHeadDim, "o_proj (input slice of this rank)");
        check_weight_shape(gate_up, 2 * (int64_t)d->f, H, "gate_up (gate rows, then up rows of this rank)");
        check_weight_shape(down, H, d->f, "down_proj (input slice of this rank)");
        DecoderLayer& L = d->layers[layer];
        L.qkv = qkv;
        L.o = o;
        L.gate_up = gate_up;
        L.down = down;
    });
}

int mfqb_decoder_set_head(mfqb_decoder* d, const mfqb_weight* lm_head, const void* embedding_bf16) {
    return guarded([&] {
        if (!d || !lm_head || !embedding_bf16) fail(MFQB_ERR_ARG, "mfqb_decoder_set_head: null argument");
        check_weight_shape(lm_head, d->vshard, d->cfg.hidden, "lm_head (vocabulary rows of this rank)");
        d->lm_head = lm_head;
        d->embedding = embedding_bf16;
    });
}

int mfqb_decoder_vocab_shard(const mfqb_decoder* d, int* begin, int* rows) {
    return guarded([&] {
        if (!d || !begin || !rows) fail(MFQB_ERR_ARG, "mfqb_decoder_vocab_shard: null argument");
        *begin = d->vbase;
        *rows = d->vshard;
    });
}

int mfqb_decoder_fill_cache(mfqb_decoder* d, int ctx_len, unsigned seed, mfqb_stream_t stream) {
    return guarded([&] {
        if (!d || ctx_len < 0 || ctx_len >= d->cfg.max_ctx) fail(MFQB_ERR_ARG, "mfqb_decoder_fill_cache: context length must be in [0, max_ctx)");
        DeviceGuard guard(d->device);
        unsigned s = seed;
        for (auto& L : d->layers) {
            const size_t n = L.kcache.bytes / 2;
            fill_cache_kernel<<<1024, 256, 0, stream>>>(static_cast<__nv_bfloat16*>(L.kcache.p), n, s++);
            fill_cache_kernel<<<1024, 256, 0, stream>>>(static_cast<__nv_bfloat16*>(L.vcache.p), n, s++);
        }
        std::vector<int> pos((size_t)d->cfg.max_batch, ctx_len);
        MFQB_CUDA(cudaMemcpyAsync(d->pos.p, pos.data(), pos.size() * 4, cudaMemcpyHostToDevice, stream));
        MFQB_CUDA(cudaStreamSynchronize(stream));
    });
}

int mfqb_decoder_step(mfqb_decoder* d, const int32_t* ids_in, int batch, int32_t* ids_out, mfqb_stream_t stream) {
    return guarded([&] {
        if (!d || !ids_in || !ids_out) fail(MFQB_ERR_ARG, "mfqb_decoder_step: null argument");
        if (batch < 1 || batch > d->cfg.max_batch) fail(MFQB_ERR_ARG, "mfqb_decoder_step: batch %d outside [1, %d]", batch, d->cfg.max_batch);
        if (!d->lm_head || !d->embedding) fail(MFQB_ERR_ARG, "mfqb_decoder_step: head weights are not set");
        for (const auto& L : d->layers)
            if (!L.qkv) fail(MFQB_ERR_ARG, "mfqb_decoder_step: a layer has no weights");
        DeviceGuard guard(d->device);
        cudaStream_t s = stream;
        const int H = d->cfg.hidden;
        launch_dep(embed_rows_kernel, dim3(batch), dim3(1024), s, static_cast<const int*>(ids_in), static_cast<const __nv_bfloat16*>(d->embedding),
                   static_cast<float*>(d->h.p), H, d->cfg.vocab);
        launch_rope_table(d, batch, s);
        const float* delta = nullptr;
        for (int li = 0; li < d->cfg.layers; ++li) delta = layer_forward(d, li, batch, delta, s);
        bool fused_head = batch == 1 && d->fused_norm;
        if (fused_head) {
            const int rc = mfqb_mul_mat_rmsnorm(d->lm_head, static_cast<const float*>(d->h.p), delta, static_cast<const float*>(d->gamma_final.p),
                                                d->cfg.rms_eps, nullptr, d->logits.p, MFQB_F32, 0, s);
            if (rc == MFQB_ERR_UNSUPPORTED) fused_head = false;
            else if (rc != MFQB_OK) throw Error(rc, mfqb_last_error());
        }
        if (!fused_head) {
            launch_dep(add_rmsnorm_kernel, dim3(batch), dim3(1024), s, static_cast<float*>(d->h.p), delta, static_cast<const float*>(d->gamma_final.p),
                       static_cast<__nv_bfloat16*>(d->xn.p), H, d->cfg.rms_eps);
            mul_mat(d->lm_head, d->xn.p, batch, d->logits.p, s);
        }
        launch_dep(argmax_slices_kernel, dim3(kArgmaxSlices, batch), dim3(256), s, static_cast<const float*>(d->logits.p), d->vshard,
                   static_cast<float*>(d->part_val.p), static_cast<int*>(d->part_idx.p));
        launch_dep(argmax_merge_kernel, dim3(batch), dim3(32), s, static_cast<const float*>(d->part_val.p), static_cast<const int*>(d->part_idx.p),
                   d->vbase, static_cast<float*>(d->best_val.p), static_cast<int*>(d->best_idx.p));
        if (d->world == 1) {
            MFQB_CUDA(cudaMemcpyAsync(ids_out, d->best_idx.p, (size_t)batch * 4, cudaMemcpyDeviceToDevice, s));
        } else {
            const int n = d->world * batch * 2;
            launch_dep(argmax_pack_kernel, dim3((n + 255) / 256), dim3(256), s, static_cast<const float*>(d->best_val.p),
                       static_cast<const int*>(d->best_idx.p), d->rank, d->world, batch, static_cast<float*>(d->gathered.p));
            const float* g = rank_sum(d, static_cast<const float*>(d->gathered.p), static_cast<float*>(d->gathered_sum.p), (size_t)n, s);
            launch_dep(argmax_pick_kernel, dim3((batch + 127) / 128), dim3(128), s, g, d->world, batch, static_cast<int*>(ids_out));
        }
        launch_dep(add_one_kernel, dim3((batch + 127) / 128), dim3(128), s, static_cast<int*>(d->pos.p), batch);
    });
}

// One block only, for parity checks: h_in [rows, H] float32 -> h_out = the residual stream after
// block `layer` (attention and FFN added), computed at the cache positions currently set.
int mfqb_decoder_layer(mfqb_decoder* d, int layer, const float* h_in, int rows, float* h_out, mfqb_stream_t stream) {
    return guarded([&] {
        if (!d || !h_in || !h_out || layer < 0 || layer >= d->cfg.layers || rows < 1 || rows > d->cfg.max_batch)
            fail(MFQB_ERR_ARG, "mfqb_decoder_layer: bad argument");
        DeviceGuard guard(d->device);
        const size_t bytes = (size_t)rows * d->cfg.hidden * 4;
        MFQB_CUDA(cudaMemcpyAsync(d->h.p, h_in, bytes, cudaMemcpyDeviceToDevice, stream));
        launch_rope_table(d, rows, stream);
        const float* delta = layer_forward(d, layer, rows, nullptr, stream);
        // fold the FFN output in with a norm whose bf16 output is discarded
        launch_dep(add_rmsnorm_kernel, dim3(rows), dim3(1024), stream, static_cast<float*>(d->h.p), delta, static_cast<const float*>(d->gamma_final.p),
                   static_cast<__nv_bfloat16*>(d->xn.p), d->cfg.hidden, d->cfg.rms_eps);
        MFQB_CUDA(cudaMemcpyAsync(h_out, d->h.p, bytes, cudaMemcpyDeviceToDevice, stream));
    });
}

// Copies the logits of the last step, this rank's vocabulary rows: out [rows, shard rows] float32.
int mfqb_decoder_read_logits(const mfqb_decoder* d, int rows, float* out, mfqb_stream_t stream) {
    return guarded([&] {
        if (!d || !out || rows < 1 || rows > d->cfg.max_batch) fail(MFQB_ERR_ARG, "mfqb_decoder_read_logits: bad argument");
        DeviceGuard guard(d->device);
        MFQB_CUDA(cudaMemcpyAsync(out, d->logits.p, (size_t)rows * d->vshard * 4, cudaMemcpyDeviceToDevice, stream));
    });
}

// Reads back one layer's cache rows [nkv_local][ctx][128] of sequence `row` (bf16), for parity checks.
int mfqb_decoder_read_cache(const mfqb_decoder* d, int layer, int row, int which, int ctx, void* out_bf16, mfqb_stream_t stream) {
    return guarded([&] {
        if (!d || !out_bf16 || layer < 0 || layer >= d->cfg.layers || row < 0 || row >= d->cfg.max_batch || ctx < 0 || ctx > d->cfg.max_ctx)
            fail(MFQB_ERR_ARG, "mfqb_decoder_read_cache: bad argument");
        DeviceGuard guard(d->device);
        const DecoderLayer& L = d->layers[layer];
        const char* base = static_cast<const char*>(which ? L.vcache.p : L.kcache.p);
        for (int hh = 0; hh < d->nkv; ++hh)
            MFQB_CUDA(cudaMemcpyAsync(static_cast<char*>(out_bf16) + (size_t)hh * ctx * kHeadDim * 2,
                                      base + (((size_t)row * d->nkv + hh) * d->cfg.max_ctx) * kHeadDim * 2, (size_t)ctx * kHeadDim * 2,
                                      cudaMemcpyDeviceToDevice, stream));
    });
}

int mfqb_decoder_free(mfqb_decoder* d) {
    return guarded([&] {
        if (!d) return;
        DeviceGuard guard(d->device);
        delete d;
    });
}

#pragma GCC visibility pop
}  // extern "C"
