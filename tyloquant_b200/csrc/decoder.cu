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
static void launch_dep(void (*kernel)(KArgs...), dim3 grid, dim3 block, cudaStream_t s, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = 0;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    MFQB_CUDA(cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...));
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

// qkv [rows, (nq + 2 nkv) * 128] float32 -> rotary embedding on q and k (halves convention: pairs
// (i, i + 64)), q kept as float32 pre-scaled by 1/sqrt(128), k and v written as bf16 into the cache
// at position pos[row].  Cache layout: [rows][nkv][max_ctx][128] for K and for V.
__global__ void __launch_bounds__(64) rope_kv_write_kernel(const float* __restrict__ qkv, const int* __restrict__ pos, float* __restrict__ q_out,
                                                           __nv_bfloat16* __restrict__ kcache, __nv_bfloat16* __restrict__ vcache, int nq, int nkv,
                                                           int max_ctx, float theta) {
    dep_wait();
    const int row = blockIdx.y, head = blockIdx.x, i = threadIdx.x;   // 64 threads: one rotation pair each
    const int p = pos[row];
    const float* src = qkv + ((size_t)row * (nq + 2 * nkv) + head) * kHeadDim;
    const float a = src[i], b = src[i + 64];
    if (head >= nq + nkv) {   // value head: plain copy into the cache
        __nv_bfloat16* dst = vcache + (((size_t)row * nkv + (head - nq - nkv)) * max_ctx + p) * kHeadDim;
        dst[i] = __float2bfloat16_rn(a);
        dst[i + 64] = __float2bfloat16_rn(b);
        return;
    }
    const float freq = powf(theta, -(float)(2 * i) / (float)kHeadDim);
    float sn, cs;
    sincosf((float)p * freq, &sn, &cs);
    const float ra = a * cs - b * sn, rb = b * cs + a * sn;
    if (head < nq) {
        float* dst = q_out + ((size_t)row * nq + head) * kHeadDim;
        const float scale = 0.08838834764831845f;   // 1 / sqrt(128)
        dst[i] = ra * scale;
        dst[i + 64] = rb * scale;
    } else {
        __nv_bfloat16* dst = kcache + (((size_t)row * nkv + (head - nq)) * max_ctx + p) * kHeadDim;
        dst[i] = __float2bfloat16_rn(ra);
        dst[i + 64] = __float2bfloat16_rn(rb);
    }
}

// Grouped-query decode attention, first pass: CTA (split, kv head, row) scans its slice of the cache for
// the G = nq / nkv query heads that share the KV head.  A half-warp holds one token (16 lanes x 8
// dimensions = one 16-byte load per lane for K and for V); the CTA's eight half-warps take tokens
// round robin, two tokens per half-warp and iteration, so that four 16-byte loads per lane are in
// flight.  Scores are reduced inside the half-warp, the soft-max runs online per half-warp and
// head.  Writes (max, sum, unnormalised output[128]) per (row, query head, split).
__device__ __forceinline__ void bf16x8_to_f32(const uint4& r, float* f) {
    f[0] = __uint_as_float(r.x << 16); f[1] = __uint_as_float(r.x & 0xFFFF0000u);
    f[2] = __uint_as_float(r.y << 16); f[3] = __uint_as_float(r.y & 0xFFFF0000u);
    f[4] = __uint_as_float(r.z << 16); f[5] = __uint_as_float(r.z & 0xFFFF0000u);
    f[6] = __uint_as_float(r.w << 16); f[7] = __uint_as_float(r.w & 0xFFFF0000u);
}
template <int G>
__global__ void __launch_bounds__(128) attn_decode_partial_kernel(const float* __restrict__ q, const __nv_bfloat16* __restrict__ kcache,
                                                                  const __nv_bfloat16* __restrict__ vcache, const int* __restrict__ pos,
                                                                  float* __restrict__ part, int nq, int nkv, int max_ctx, int nsplit) {
    dep_wait();
    const int split = blockIdx.x, kvh = blockIdx.y, row = blockIdx.z;
    const int lane = threadIdx.x & 31, l16 = lane & 15, slot = threadIdx.x >> 4;   // slot: half-warp 0..7 of the CTA
    const int len = pos[row] + 1;   // the token written by this step takes part
    const int per = (len + nsplit - 1) / nsplit;
    const int t0 = split * per, t1 = min(len, t0 + per);
    float qv[G][8];
#pragma unroll
    for (int g = 0; g < G; ++g) {
        const float4* src = reinterpret_cast<const float4*>(q + ((size_t)row * nq + kvh * G + g) * kHeadDim + 8 * l16);
        const float4 a = src[0], b = src[1];
        qv[g][0] = a.x; qv[g][1] = a.y; qv[g][2] = a.z; qv[g][3] = a.w;
        qv[g][4] = b.x; qv[g][5] = b.y; qv[g][6] = b.z; qv[g][7] = b.w;
    }
    float m[G], l[G], acc[G][8];
#pragma unroll
    for (int g = 0; g < G; ++g) {
        m[g] = -INFINITY;
        l[g] = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[g][i] = 0.f;
    }
    const __nv_bfloat16* kb = kcache + ((size_t)row * nkv + kvh) * max_ctx * kHeadDim + 8 * l16;
    const __nv_bfloat16* vb = vcache + ((size_t)row * nkv + kvh) * max_ctx * kHeadDim + 8 * l16;
    const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
    for (int base = t0; base < t1; base += 16) {   // uniform trip count over the CTA: the shuffles below need whole warps
        const int ta = base + slot, tb = ta + 8;
        const bool va = ta < t1, vb2 = tb < t1;
        const uint4 kra = va ? *reinterpret_cast<const uint4*>(kb + (size_t)ta * kHeadDim) : zero;
        const uint4 krb = vb2 ? *reinterpret_cast<const uint4*>(kb + (size_t)tb * kHeadDim) : zero;
        const uint4 vra = va ? *reinterpret_cast<const uint4*>(vb + (size_t)ta * kHeadDim) : zero;
        const uint4 vrb = vb2 ? *reinterpret_cast<const uint4*>(vb + (size_t)tb * kHeadDim) : zero;
        float ka[8], kbv[8], fa[8], fb[8];
        bf16x8_to_f32(kra, ka);
        bf16x8_to_f32(krb, kbv);
        bf16x8_to_f32(vra, fa);
        bf16x8_to_f32(vrb, fb);
        float sa[G], sb[G];
#pragma unroll
        for (int g = 0; g < G; ++g) {
            float x = 0.f, y = 0.f;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                x += qv[g][i] * ka[i];
                y += qv[g][i] * kbv[i];
            }
            sa[g] = x;
            sb[g] = y;
        }
#pragma unroll
        for (int o = 8; o > 0; o >>= 1)
#pragma unroll
            for (int g = 0; g < G; ++g) {
                sa[g] += __shfl_xor_sync(0xffffffffu, sa[g], o);
                sb[g] += __shfl_xor_sync(0xffffffffu, sb[g], o);
            }
        if (va) {   // uniform over the half-warp; tb valid implies ta valid
#pragma unroll
            for (int g = 0; g < G; ++g) {
                const float s1 = vb2 ? sb[g] : -INFINITY;
                const float mn = fmaxf(m[g], fmaxf(sa[g], s1));
                const float corr = __expf(m[g] - mn), pa = __expf(sa[g] - mn), pb = __expf(s1 - mn);
                l[g] = l[g] * corr + pa + pb;
#pragma unroll
                for (int i = 0; i < 8; ++i) acc[g][i] = acc[g][i] * corr + pa * fa[i] + pb * fb[i];
                m[g] = mn;
            }
        }
    }
    // the eight half-warps of the CTA meet in shared memory
    __shared__ float sm_m[8][G], sm_l[8][G];
    __shared__ __align__(16) float sm_acc[8][G][kHeadDim];
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
        float* dst = part + (((size_t)row * nq + kvh * G + g) * nsplit + split) * (kHeadDim + 2);
        if (d == 0) { dst[0] = mm; dst[1] = ll; }
        dst[2 + d] = aa;
    }
}

// Second pass: merges the splits of one (row, query head) and writes the bf16 attention output.
__global__ void __launch_bounds__(128) attn_decode_merge_kernel(const float* __restrict__ part, __nv_bfloat16* __restrict__ out, int nq, int nsplit) {
    dep_wait();
    const int head = blockIdx.x, row = blockIdx.y, d = threadIdx.x;
    const float* src = part + ((size_t)row * nq + head) * nsplit * (kHeadDim + 2);
    float mm = -INFINITY;
    for (int s = 0; s < nsplit; ++s) mm = fmaxf(mm, src[(size_t)s * (kHeadDim + 2)]);
    float ll = 0.f, aa = 0.f;
    for (int s = 0; s < nsplit; ++s) {
        const float ms = src[(size_t)s * (kHeadDim + 2)];
        const float c = ms == -INFINITY ? 0.f : __expf(ms - mm);
        ll += src[(size_t)s * (kHeadDim + 2) + 1] * c;
        aa += src[(size_t)s * (kHeadDim + 2) + 2 + d] * c;
    }
    out[((size_t)row * nq + head) * kHeadDim + d] = __float2bfloat16_rn(aa / ll);
}

// gate_up [rows, 2F] float32 (gate columns first) -> act = up * gate / (1 + exp(-gate)) as bf16 [rows, F]
// (mfq/kernels/cuda/glu.cuh:6-17).
__global__ void swiglu_rows_kernel(const float* __restrict__ gu, __nv_bfloat16* __restrict__ act, int rows, int F) {
    dep_wait();
    const size_t total = (size_t)rows * F;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const size_t r = i / F, c = i % F;
        const float g = gu[r * 2 * F + c], u = gu[r * 2 * F + F + c];
        act[i] = __float2bfloat16_rn(u * g / (1.f + __expf(-g)));
    }
}

// logits [rows, n] float32 -> (largest value, its index + index_base) per row; ties go to the smaller index.
__global__ void __launch_bounds__(1024) argmax_rows_kernel(const float* __restrict__ logits, int n, int index_base, float* __restrict__ best_val,
                                                           int* __restrict__ best_idx) {
    dep_wait();
    __shared__ float sv[32];
    __shared__ int si[32];
    const float* row = logits + (size_t)blockIdx.x * n;
    float bv = -INFINITY;
    int bi = 0x7FFFFFFF;
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        const float v = row[i];
        if (v > bv || (v == bv && i < bi)) { bv = v; bi = i; }
    }
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    if ((threadIdx.x & 31) == 0) { sv[threadIdx.x >> 5] = bv; si[threadIdx.x >> 5] = bi; }
    __syncthreads();
    if (threadIdx.x < 32) {
        bv = threadIdx.x < (blockDim.x >> 5) ? sv[threadIdx.x] : -INFINITY;
        bi = threadIdx.x < (blockDim.x >> 5) ? si[threadIdx.x] : 0x7FFFFFFF;
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
        }
        if (threadIdx.x == 0) { best_val[blockIdx.x] = bv; best_idx[blockIdx.x] = bi + index_base; }
    }
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
    for (int i = threadIdx.x; i < H; i += blockDim.x) h[(size_t)r * H + i] = __bfloat162float(table[(size_t)id * H + i]);
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
    int nq = 0, nkv = 0, f = 0, vshard = 0, vbase = 0, sms = 0;
    std::vector<DecoderLayer> layers;
    const mfqb_weight* lm_head = nullptr;
    const void* embedding = nullptr;   // bf16 [vocab, H] on the device, borrowed
    DevBuf gamma_final;
    // workspaces
    DevBuf h, xn, qkv, q, attn, proj, proj_sum, gu, act, logits, part, best_val, best_idx, gathered, gathered_sum, pos;
};

// Context splits of the decode attention: enough CTAs to fill every SM about four times over, each
// split at least one round of the CTA's half-warps.
constexpr int kMaxSplits = 64;
static int attn_splits(const mfqb_decoder* d, int rows) {
    const int want = (4 * d->sms + d->nkv * rows - 1) / (d->nkv * rows);
    return std::max(1, std::min(kMaxSplits, want));
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
    launch_dep(add_rmsnorm_kernel, dim3(rows), dim3(1024), s, static_cast<float*>(d->h.p), delta, static_cast<const float*>(L.gamma_attn.p),
               static_cast<__nv_bfloat16*>(d->xn.p), H, d->cfg.rms_eps);
    mul_mat(L.qkv, d->xn.p, rows, d->qkv.p, s);
    launch_dep(rope_kv_write_kernel, dim3(d->nq + 2 * d->nkv, rows), dim3(64), s, static_cast<const float*>(d->qkv.p),
               static_cast<const int*>(d->pos.p), static_cast<float*>(d->q.p), static_cast<__nv_bfloat16*>(L.kcache.p),
               static_cast<__nv_bfloat16*>(L.vcache.p), d->nq, d->nkv, d->cfg.max_ctx, d->cfg.rope_theta);
    const int nsplit = attn_splits(d, rows);
    const dim3 agrid(nsplit, d->nkv, rows);
    const float* qp = static_cast<const float*>(d->q.p);
    const __nv_bfloat16 *kc = static_cast<const __nv_bfloat16*>(L.kcache.p), *vc = static_cast<const __nv_bfloat16*>(L.vcache.p);
    const int* pos = static_cast<const int*>(d->pos.p);
    float* part = static_cast<float*>(d->part.p);
    switch (G) {
        case 1: launch_dep(attn_decode_partial_kernel<1>, agrid, dim3(128), s, qp, kc, vc, pos, part, d->nq, d->nkv, d->cfg.max_ctx, nsplit); break;
        case 2: launch_dep(attn_decode_partial_kernel<2>, agrid, dim3(128), s, qp, kc, vc, pos, part, d->nq, d->nkv, d->cfg.max_ctx, nsplit); break;
        case 4: launch_dep(attn_decode_partial_kernel<4>, agrid, dim3(128), s, qp, kc, vc, pos, part, d->nq, d->nkv, d->cfg.max_ctx, nsplit); break;
        case 8: launch_dep(attn_decode_partial_kernel<8>, agrid, dim3(128), s, qp, kc, vc, pos, part, d->nq, d->nkv, d->cfg.max_ctx, nsplit); break;
        default: fail(MFQB_ERR_UNSUPPORTED, "query heads per KV head must be 1, 2, 4 or 8, got %d", G);
    }
    launch_dep(attn_decode_merge_kernel, dim3(d->nq, rows), dim3(128), s, static_cast<const float*>(part), static_cast<__nv_bfloat16*>(d->attn.p),
               d->nq, nsplit);
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
    launch_dep(add_rmsnorm_kernel, dim3(rows), dim3(1024), s, static_cast<float*>(d->h.p), o_out, static_cast<const float*>(L.gamma_ffn.p),
               static_cast<__nv_bfloat16*>(d->xn.p), H, d->cfg.rms_eps);
    mul_mat(L.gate_up, d->xn.p, rows, d->gu.p, s);
    if (d->world == 1 && rows == 1) {   // the down projection computes the activation as it loads its row
        const int rc = mfqb_mul_mat_swiglu(L.down, d->gu.p, 1, d->proj.p, MFQB_F32, s);
        if (rc != MFQB_OK) throw Error(rc, mfqb_last_error());
        return static_cast<const float*>(d->proj.p);
    }
    launch_dep(swiglu_rows_kernel, dim3(std::min(1024, (rows * d->f + 255) / 256)), dim3(256), s, static_cast<const float*>(d->gu.p),
               static_cast<__nv_bfloat16*>(d->act.p), rows, d->f);
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
            cfg->hidden != cfg->n_q_heads * kHeadDim || cfg->hidden % 8)
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
        d->xn.alloc(B * H * 2);
        d->qkv.alloc(B * (d->nq + 2 * d->nkv) * kHeadDim * 4);
        d->q.alloc(B * d->nq * kHeadDim * 4);
        d->attn.alloc(B * d->nq * kHeadDim * 2);
        d->proj.alloc(B * H * 4);
        d->proj_sum.alloc(B * H * 4);
        d->gu.alloc(B * 2 * d->f * 4);
        d->act.alloc(B * d->f * 2);
        d->logits.alloc(B * std::max(d->vshard, 1) * 4);
        d->part.alloc(B * d->nq * kMaxSplits * (kHeadDim + 2) * 4);
        d->best_val.alloc(B * 4);
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
        launch_dep(embed_rows_kernel, dim3(batch), dim3(256), s, static_cast<const int*>(ids_in), static_cast<const __nv_bfloat16*>(d->embedding),
                   static_cast<float*>(d->h.p), H, d->cfg.vocab);
        const float* delta = nullptr;
        for (int li = 0; li < d->cfg.layers; ++li) delta = layer_forward(d, li, batch, delta, s);
        launch_dep(add_rmsnorm_kernel, dim3(batch), dim3(1024), s, static_cast<float*>(d->h.p), delta, static_cast<const float*>(d->gamma_final.p),
                   static_cast<__nv_bfloat16*>(d->xn.p), H, d->cfg.rms_eps);
        mul_mat(d->lm_head, d->xn.p, batch, d->logits.p, s);
        launch_dep(argmax_rows_kernel, dim3(batch), dim3(1024), s, static_cast<const float*>(d->logits.p), d->vshard, d->vbase,
                   static_cast<float*>(d->best_val.p), static_cast<int*>(d->best_idx.p));
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
        const float* delta = layer_forward(d, layer, rows, nullptr, stream);
        // fold the FFN output in with a norm whose bf16 output is discarded
        launch_dep(add_rmsnorm_kernel, dim3(rows), dim3(1024), stream, static_cast<float*>(d->h.p), delta, static_cast<const float*>(d->gamma_final.p),
                   static_cast<__nv_bfloat16*>(d->xn.p), d->cfg.hidden, d->cfg.rms_eps);
        MFQB_CUDA(cudaMemcpyAsync(h_out, d->h.p, bytes, cudaMemcpyDeviceToDevice, stream));
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
