// Dense weight handles: blob -> device layout -> decode / multiply entry points.
#include <cuda_bf16.h>

#include <algorithm>
#include <memory>
#include <mutex>

#include "cuda_util.h"
#include "nint_gemm_tc.cuh"
#include "nint_gemv_m1.cuh"
#include "nvq.h"

namespace mfqb {

int device_sm_count(int device) {
    static std::mutex mu;
    static int cache[64] = {0};
    std::lock_guard<std::mutex> lock(mu);
    if (device < 0 || device >= 64) fail(MFQB_ERR_ARG, "device index %d out of range", device);
    if (!cache[device]) {
        int v = 0;
        MFQB_CUDA(cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, device));
        cache[device] = v;
    }
    return cache[device];
}

GemvPlan plan_nint_gemv(const NintDev& w, int m, int num_sms) {
    GemvPlan p;
    p.grid_y = 1;
    // Two 8-warp CTAs per SM; each CTA owns whole row-blocks (all chunks of K), so partial sums
    // stay in its shared memory.
    const int target = 2 * num_sms;
    p.rb_per_cta = std::max(1, (w.nrb + target - 1) / target);
    p.grid = (w.nrb + p.rb_per_cta - 1) / p.rb_per_cta;
    const int warps = 8;
    p.threads = warps * 32;
    // x in shared memory: rows padded to whole chunks, stride chosen so that the eight batch rows a
    // warp reads together fall into distinct banks (stride in words = 2*PER mod 32), kept a
    // multiple of 8 elements for the 16-byte staging copies.
    const int kp = w.nchunks * kChunkGroups * w.gs;
    int words = (kp + 1) / 2;
    if (m > 1) words += (((2 * w.per - words) % 32) + 32) % 32;
    p.xstride = ((words * 2 + 7) / 8) * 8;
    p.stages = 0;
    if (m == 1) {   // single-row kernel: partial sums and anchors [rb][16], x, and a record ring per warp
        const size_t rec_bytes = (size_t)w.rec_words * 4;
        p.stages = gemv_m1_stages(w.rec_words);
        // three CTAs per SM, all resident at once; row-blocks are split evenly inside the kernel
        p.grid = std::min(w.nrb, 3 * num_sms);
        p.rb_per_cta = (w.nrb + p.grid - 1) / p.grid;
        p.smem = (size_t)p.rb_per_cta * 16 * 8 + (size_t)p.xstride * 2 + (size_t)w.nchunks * kChunkGroups * 4 +
                 (size_t)warps * p.stages * rec_bytes;
        return p;
    }
    const size_t fixed = (size_t)p.rb_per_cta * 128 * 4 + (size_t)warps * 64 * 4;
    const size_t xbytes = (size_t)m * p.xstride * 2;
    if (fixed + xbytes > 100 * 1024) p.xstride = 0;   // too long to stage twice per SM: read x from global
    p.smem = fixed + (p.xstride ? xbytes : 0);
    return p;
}

// ---- reference decoder on the GPU -----------------------------------------------------------
// One thread per (row, group, lane-of-quad): reads its code pairs and the two scale fields
// through the same accessors as the GEMV and writes w = fl(fl(d*q) - m), d = fl(ns*ss),
// m = fl(nm*sm): three separately rounded float32 operations, as the reference decoder does
// (mfq/quantize/nint_quant.py:896-908).
template <int SW>
__device__ __forceinline__ void read_scales(const NintDev& w, size_t item, int q, int r, int g, float& ss, float& sm) {
    constexpr int SWC = PairUnit<SW>::words_for(16);
    uint32_t sq[SWC];
#pragma unroll
    for (int i = 0; i < SWC; ++i) sq[i] = w.items[item * w.rec_words + w.wc * 32 + i * 8 + q];
    const uint32_t sp = PairUnit<SW>::get_rt(sq + (g / PairUnit<SW>::NP) * PairUnit<SW>::U, g % PairUnit<SW>::NP);
    const int mt = 8 + 4 * r + g / 2;
    const uint32_t mp = PairUnit<SW>::get_rt(sq + (mt / PairUnit<SW>::NP) * PairUnit<SW>::U, mt % PairUnit<SW>::NP);
    ss = (float)(r ? (sp >> 16) : (sp & 0xFFFFu));
    sm = (float)((g & 1) ? (mp >> 16) : (mp & 0xFFFFu));
}

template <int BITS>
__global__ void nint_dequant_kernel(const NintDev w, void* out, int out_dtype) {
    using QU = PairUnit<BITS>;
    const size_t total = (size_t)w.n * w.ng * 4;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
        const int c = (int)(idx & 3);
        const size_t rg = idx >> 2;
        const int grp = (int)(rg % w.ng), row = (int)(rg / w.ng);
        const int rb = row >> 4, q = row & 7, r = (row >> 3) & 1, ch = grp / kChunkGroups, g = grp % kChunkGroups;
        const int lane = 4 * q + c, half = w.per / 2;
        const size_t item = (size_t)rb * w.nchunks + ch;
        float ss, sm;
        switch (w.sw) {
            case 5: read_scales<5>(w, item, q, r, g, ss, sm); break;
            case 6: read_scales<6>(w, item, q, r, g, ss, sm); break;
            case 7: read_scales<7>(w, item, q, r, g, ss, sm); break;
            default: read_scales<8>(w, item, q, r, g, ss, sm); break;
        }
        const uint32_t an = w.anchors[row];
        const float2 nsm = __half22float2(*reinterpret_cast<const __half2*>(&an));
        const float d = __fmul_rn(nsm.x, ss), m = __fmul_rn(nsm.y, sm);
        for (int j = 0; j < half; ++j) {
            const int t = (g * 2 + r) * half + j, unit = t / QU::NP;
            uint32_t uw[QU::U];
#pragma unroll
            for (int u = 0; u < QU::U; ++u) uw[u] = w.items[item * w.rec_words + (unit * QU::U + u) * 32 + lane];
            const uint32_t pr = QU::get_rt(uw, t % QU::NP);
            const int i0 = c * w.per + 2 * j, k0 = grp * w.gs + i0;
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                if (i0 + e < w.gs && k0 + e < w.k) {
                    const float code = (float)(e ? (pr >> 16) : (pr & 0xFFFFu));
                    const float v = __fsub_rn(__fmul_rn(d, code), m);
                    const size_t o = (size_t)row * w.k + k0 + e;
                    if (out_dtype == MFQB_F32) reinterpret_cast<float*>(out)[o] = v;
                    else reinterpret_cast<__nv_bfloat16*>(out)[o] = __float2bfloat16_rn(v);
                }
            }
        }
    }
}

static void launch_nint_dequant(const NintDev& w, void* out, int out_dtype, cudaStream_t s) {
    const size_t total = (size_t)w.n * w.ng * 4;
    const int block = 256;
    const int grid = (int)std::min<size_t>((total + block - 1) / block, 148 * 32);
    switch (w.bits) {
        case 2: nint_dequant_kernel<2><<<grid, block, 0, s>>>(w, out, out_dtype); break;
        case 3: nint_dequant_kernel<3><<<grid, block, 0, s>>>(w, out, out_dtype); break;
        case 4: nint_dequant_kernel<4><<<grid, block, 0, s>>>(w, out, out_dtype); break;
        case 5: nint_dequant_kernel<5><<<grid, block, 0, s>>>(w, out, out_dtype); break;
        case 6: nint_dequant_kernel<6><<<grid, block, 0, s>>>(w, out, out_dtype); break;
        case 8: nint_dequant_kernel<8><<<grid, block, 0, s>>>(w, out, out_dtype); break;
        default: fail(MFQB_ERR_UNSUPPORTED, "NINT%d has no kernel", w.bits);
    }
    MFQB_CUDA(cudaGetLastError());
}

static void launch_nint_gemv(const NintDev& w, const void* x, int m, void* y, int y_dtype, int ldy, int device,
                             cudaStream_t s) {
    GemvArgs a;
    a.w = w;
    a.x = static_cast<const __nv_bfloat16*>(x);
    a.y = y;
    a.m = m;
    a.ldy = ldy;
    a.y_dtype = y_dtype;
    a.route_ids = nullptr;
    a.expert_pool = a.expert_local = nullptr;
    a.pool = a.rb_per_expert = a.routes = a.x_per_pair = 0;
    a.expert_bounds = a.tile_bounds = a.pair_order = nullptr;
    a.n_experts = 0;
    const GemvPlan p = plan_nint_gemv(w, m, device_sm_count(device));
    a.rb_per_cta = p.rb_per_cta;
    a.xstride = p.xstride;
    a.stages = p.stages;
    cudaError_t e;
    switch (w.bits) {
        case 2: e = launch_nint_gemv_bits<2>(a, p, s); break;
        case 3: e = launch_nint_gemv_bits<3>(a, p, s); break;
        case 4: e = launch_nint_gemv_bits<4>(a, p, s); break;
        case 5: e = launch_nint_gemv_bits<5>(a, p, s); break;
        case 6: e = launch_nint_gemv_bits<6>(a, p, s); break;
        case 8: e = launch_nint_gemv_bits<8>(a, p, s); break;
        default: fail(MFQB_ERR_UNSUPPORTED, "NINT%d has no kernel", w.bits);
    }
    if (e != cudaSuccess) fail(MFQB_ERR_CUDA, "NINT%d gs=%d GEMV launch: %s", w.bits, w.gs, cudaGetErrorString(e));
}

// Routed single-row launch over (splits, pairs) CTAs for one cohort; see GemvArgs.
void launch_nint_gemv_routed(GemvArgs a, int pairs, int device, cudaStream_t s) {
    const NintDev& w = a.w;
    a.m = 1;
    GemvPlan p = plan_nint_gemv(w, 1, device_sm_count(device));
    const int want = (3 * device_sm_count(device) + pairs - 1) / std::max(pairs, 1);
    const int splits = std::max(1, std::min(a.rb_per_expert, want));
    p.rb_per_cta = (a.rb_per_expert + splits - 1) / splits;
    p.smem = (size_t)p.rb_per_cta * 16 * 8 + (size_t)p.xstride * 2 + (size_t)w.nchunks * kChunkGroups * 4 +
             (size_t)8 * p.stages * w.rec_words * 4;
    a.rb_per_cta = p.rb_per_cta;
    a.xstride = p.xstride;
    a.stages = p.stages;
    p.grid = splits;
    p.grid_y = pairs;
    cudaError_t e;
    switch (w.bits) {
        case 2: e = launch_nint_gemv_bits<2>(a, p, s); break;
        case 3: e = launch_nint_gemv_bits<3>(a, p, s); break;
        case 4: e = launch_nint_gemv_bits<4>(a, p, s); break;
        case 5: e = launch_nint_gemv_bits<5>(a, p, s); break;
        case 6: e = launch_nint_gemv_bits<6>(a, p, s); break;
        case 8: e = launch_nint_gemv_bits<8>(a, p, s); break;
        default: fail(MFQB_ERR_UNSUPPORTED, "NINT%d has no kernel", w.bits);
    }
    if (e != cudaSuccess) fail(MFQB_ERR_CUDA, "NINT%d routed GEMV launch: %s", w.bits, cudaGetErrorString(e));
}

// ---- tcgen05 prefill GEMM: x conversion pre-pass, per-device scratch and status word -----------
__global__ void x_to_f16_kernel(const __nv_bfloat16* __restrict__ x, int m, int k, int kx, __half* __restrict__ out) {
    const size_t total = (size_t)m * kx;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const size_t r = i / kx, c = i % kx;
        // bf16 -> f16: exact for |x| in [2^-14, 65504]; larger magnitudes saturate to +-65504
        float v = c < (size_t)k ? __bfloat162float(x[r * k + c]) : 0.f;
        v = fminf(fmaxf(v, -65504.f), 65504.f);
        out[i] = __float2half_rn(v);
    }
}

struct GemmDeviceState {
    std::mutex mu;
    DevBuf x16[64];
    int* status_host[64] = {nullptr};
    int* status_dev[64] = {nullptr};
};
static GemmDeviceState g_gemm;

static int* gemm_status_word(int device) {   // pinned, mapped: the host can read it without a sync
    if (!g_gemm.status_host[device]) {
        MFQB_CUDA(cudaHostAlloc((void**)&g_gemm.status_host[device], sizeof(int), cudaHostAllocMapped));
        *g_gemm.status_host[device] = 0;
        MFQB_CUDA(cudaHostGetDevicePointer((void**)&g_gemm.status_dev[device], g_gemm.status_host[device], 0));
    }
    return g_gemm.status_dev[device];
}

// Tensor map of the f16 activations [m, kx] for 64-column x bn-row boxes with the 128-byte swizzle.
// cuTensorMapEncodeTiled is looked up through the runtime, so the library links only libcudart.
static CUtensorMap make_x_map(const void* x16, int m, int kx, int bn) {
    typedef CUresult (*EncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                 const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                 CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
    static EncodeFn encode = nullptr;
    if (!encode) {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult qres;
        MFQB_CUDA(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres));
        if (!fn || qres != cudaDriverEntryPointSuccess) fail(MFQB_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
        encode = reinterpret_cast<EncodeFn>(fn);
    }
    CUtensorMap map;
    const cuuint64_t dims[2] = {(cuuint64_t)kx, (cuuint64_t)m};
    const cuuint64_t strides[1] = {(cuuint64_t)kx * sizeof(__half)};
    const cuuint32_t box[2] = {64u, (cuuint32_t)bn};
    const cuuint32_t elem[2] = {1u, 1u};
    const CUresult r = encode(&map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(x16), dims, strides, box, elem,
                              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) fail(MFQB_ERR_CUDA, "cuTensorMapEncodeTiled failed with code %d", (int)r);
    return map;
}

// Returns false when this weight has no tensor-core tile kernel (the caller falls back to GEMV passes).
static bool launch_nint_gemm(const NintDev& w, const void* x, int m, void* y, int y_dtype, int device, cudaStream_t s) {
    const GemmPlan p = plan_nint_gemm(w, m);
    if (p.bn == 0 || w.sw == 8) return false;
    std::lock_guard<std::mutex> lock(g_gemm.mu);
    GemmArgs a{};
    a.w = w;
    a.m = m;
    a.kx = (w.k + 7) / 8 * 8;
    a.y = y;
    a.y_dtype = y_dtype;
    a.bn = p.bn;
    a.stages = p.stages;
    a.error = gemm_status_word(device);
    DevBuf& xb = g_gemm.x16[device];
    const size_t need = (size_t)m * a.kx * sizeof(__half);
    if (xb.bytes < need) xb.alloc(need + need / 2);
    a.x16 = static_cast<const __half*>(xb.p);
    const size_t total = (size_t)m * a.kx;
    x_to_f16_kernel<<<(int)std::min<size_t>((total + 255) / 256, 148 * 8), 256, 0, s>>>(static_cast<const __nv_bfloat16*>(x), m, w.k,
                                                                                      a.kx, static_cast<__half*>(xb.p));
    MFQB_CUDA(cudaGetLastError());
    const CUtensorMap x_map = make_x_map(xb.p, m, a.kx, p.bn);
    cudaError_t e;
    switch (w.bits) {
        case 2: e = launch_nint_gemm_bits<2>(a, p, x_map, s); break;
        case 3: e = launch_nint_gemm_bits<3>(a, p, x_map, s); break;
        case 4: e = launch_nint_gemm_bits<4>(a, p, x_map, s); break;
        case 5: e = launch_nint_gemm_bits<5>(a, p, x_map, s); break;
        case 6: e = launch_nint_gemm_bits<6>(a, p, x_map, s); break;
        case 8: e = launch_nint_gemm_bits<8>(a, p, x_map, s); break;
        default: return false;
    }
    if (e == cudaErrorNotSupported) return false;
    if (e != cudaSuccess) fail(MFQB_ERR_CUDA, "NINT%d gs=%d GEMM launch: %s", w.bits, w.gs, cudaGetErrorString(e));
    return true;
}

int gemm_device_status(int device) {
    std::lock_guard<std::mutex> lock(g_gemm.mu);
    return g_gemm.status_host[device] ? *static_cast<volatile int*>(g_gemm.status_host[device]) : 0;
}

// Batched kernel over route-plan tiles (up to 8 pairs of one expert each) for one cohort.
void launch_nint_gemv_routed_tiles(GemvArgs a, int max_tiles, int device, cudaStream_t s) {
    const NintDev& w = a.w;
    a.m = 8;
    GemvPlan p = plan_nint_gemv(w, 8, device_sm_count(device));
    p.rb_per_cta = std::min(a.rb_per_expert, 48);
    const int splits = (a.rb_per_expert + p.rb_per_cta - 1) / p.rb_per_cta;
    const size_t fixed = (size_t)p.rb_per_cta * 128 * 4 + (size_t)8 * 64 * 4;
    const size_t xbytes = (size_t)8 * p.xstride * 2;
    if (fixed + xbytes > 100 * 1024) p.xstride = 0;
    p.smem = fixed + (p.xstride ? xbytes : 0);
    a.rb_per_cta = p.rb_per_cta;
    a.xstride = p.xstride;
    a.stages = 0;
    p.grid = splits;
    p.grid_y = max_tiles;
    p.threads = 256;
    cudaError_t e;
    switch (w.bits) {
        case 2: e = launch_nint_gemv_bits<2>(a, p, s); break;
        case 3: e = launch_nint_gemv_bits<3>(a, p, s); break;
        case 4: e = launch_nint_gemv_bits<4>(a, p, s); break;
        case 5: e = launch_nint_gemv_bits<5>(a, p, s); break;
        case 6: e = launch_nint_gemv_bits<6>(a, p, s); break;
        case 8: e = launch_nint_gemv_bits<8>(a, p, s); break;
        default: fail(MFQB_ERR_UNSUPPORTED, "NINT%d has no kernel", w.bits);
    }
    if (e != cudaSuccess) fail(MFQB_ERR_CUDA, "NINT%d routed tile launch: %s", w.bits, cudaGetErrorString(e));
}

void launch_nint_dequant_view(const NintDev& w, void* out, int out_dtype, cudaStream_t s) { launch_nint_dequant(w, out, out_dtype, s); }

}  // namespace mfqb

using namespace mfqb;

struct mfqb_weight {
    int family = 0, device = 0;
    mfqb_weight_info info{};
    NintDev nint{};
    DevBuf items, anchors;
    NvqDevicePtr nvq;
};

namespace mfqb {

// Batch rows one GEMV launch covers (the n8 slot of the tensor-core tile).
static int nint_gemv_max_batch(const NintDev&, int) { return 8; }

void check_nint_supported(const HostNint& t) {
    const int b = t.bits;
    if (!(b == 2 || b == 3 || b == 4 || b == 5 || b == 6 || b == 8))
        fail(MFQB_ERR_UNSUPPORTED, "NINT%d is not an executable code width (2,3,4,5,6,8)", b);
    if (t.gs % 2 || t.gs < 8 || t.gs > 64) fail(MFQB_ERR_UNSUPPORTED, "NINT groupsize %d is outside the runtime catalog", t.gs);
    const int per = nint_per(t.gs);
    const bool ok = (b == 2 && per == 4) || (b == 3 && per == 6) || (b == 4 && (per == 4 || per == 6 || per == 8 || per == 12)) ||
                    ((b == 5 || b == 8) && (per == 4 || per == 6 || per == 8 || per == 12 || per == 16)) ||
                    (b == 6 && (per == 6 || per == 8 || per == 10 || per == 12 || per == 16));
    if (!ok) fail(MFQB_ERR_UNSUPPORTED, "NINT%d with groupsize %d is outside the runtime catalog", b, t.gs);
}

static mfqb_weight* make_nint_weight(const HostNint& t, int device) {
    check_nint_supported(t);
    NintPacked p = pack_nint_device(t);
    auto w = std::make_unique<mfqb_weight>();
    DeviceGuard guard(device);
    w->family = MFQB_FAMILY_NINT;
    w->device = device;
    w->items.upload(p.items.data(), p.items.size() * 4);
    w->anchors.upload(p.anchors.data(), p.anchors.size() * 4);
    w->nint = p.d;
    w->nint.items = static_cast<const uint32_t*>(w->items.p);
    w->nint.anchors = static_cast<const uint32_t*>(w->anchors.p);
    mfqb_weight_info& i = w->info;
    i.family = MFQB_FAMILY_NINT;
    i.bits = t.bits;
    i.groupsize = t.gs;
    i.sub_bits = t.sub_bits;
    i.n = t.n;
    i.k = t.k;
    i.device = device;
    i.jsc_banks = 0;
    i.payload_bytes = nint_payload_bytes(t);
    i.device_bytes = w->items.bytes + w->anchors.bytes;
    return w.release();
}

}  // namespace mfqb

extern "C" {
#pragma GCC visibility push(default)

int mfqb_weight_from_blob_slice(const char* dtype, const void* blob, uint64_t nbytes, int axis, int64_t begin,
                                int64_t end, int device, mfqb_weight** out) {
    return guarded([&] {
        if (!dtype || !blob || !out) fail(MFQB_ERR_ARG, "mfqb_weight_from_blob: null argument");
        const std::string d(dtype);
        const bool whole = begin == 0 && end < 0;
        if (dtype_is_nint(d)) {
            HostNint t = parse_nint(blob, nbytes);
            if (d[4] - '0' != t.bits) fail(MFQB_ERR_FORMAT, "MFQ dtype/blob mismatch: %s contains NINT%d", dtype, t.bits);
            *out = whole ? make_nint_weight(t, device) : make_nint_weight(slice_nint(t, axis, begin, end), device);
        } else if (dtype_is_nvq(d)) {
            HostNvq t = parse_nvq(blob, nbytes);
            check_nvq_dtype(d, t);
            auto w = std::make_unique<mfqb_weight>();
            w->family = MFQB_FAMILY_NVQ;
            w->device = device;
            w->nvq = make_nvq_device(whole ? t : slice_nvq(t, axis, begin, end), device, &w->info);
            *out = w.release();
        } else {
            fail(MFQB_ERR_UNSUPPORTED, "dtype '%s' is outside the packed-weight execution path", dtype);
        }
    });
}

int mfqb_weight_from_blob(const char* dtype, const void* blob, uint64_t nbytes, int device, mfqb_weight** out) {
    return mfqb_weight_from_blob_slice(dtype, blob, nbytes, 0, 0, -1, device, out);
}

int mfqb_weight_info_get(const mfqb_weight* w, mfqb_weight_info* info) {
    return guarded([&] {
        if (!w || !info) fail(MFQB_ERR_ARG, "mfqb_weight_info_get: null argument");
        *info = w->info;
    });
}

int mfqb_weight_free(mfqb_weight* w) {
    return guarded([&] {
        if (!w) return;
        DeviceGuard guard(w->device);
        delete w;
    });
}

int mfqb_dequant(const mfqb_weight* w, void* out, int out_dtype, mfqb_stream_t stream) {
    return guarded([&] {
        if (!w || !out) fail(MFQB_ERR_ARG, "mfqb_dequant: null argument");
        if (out_dtype != MFQB_F32 && out_dtype != MFQB_BF16) fail(MFQB_ERR_ARG, "mfqb_dequant: bad output dtype");
        DeviceGuard guard(w->device);
        if (w->family == MFQB_FAMILY_NINT) launch_nint_dequant(w->nint, out, out_dtype, stream);
        else nvq_dequant(*w->nvq, out, out_dtype, stream);
    });
}

int mfqb_mul_mat(const mfqb_weight* w, const void* x, int m, void* y, int y_dtype, mfqb_stream_t stream) {
    return guarded([&] {
        if (!w || !x || !y) fail(MFQB_ERR_ARG, "mfqb_mul_mat: null argument");
        if (m < 1) fail(MFQB_ERR_ARG, "mfqb_mul_mat: m must be >= 1, got %d", m);
        if (y_dtype != MFQB_F32 && y_dtype != MFQB_BF16) fail(MFQB_ERR_ARG, "mfqb_mul_mat: bad output dtype");
        DeviceGuard guard(w->device);
        const int64_t n = w->info.n, k = w->info.k;
        const size_t ysz = y_dtype == MFQB_F32 ? 4 : 2;
        if (w->family == MFQB_FAMILY_NINT) {
            // more than 16 rows: tensor-core tile kernel (x conversion buffer is library scratch)
            if (m > 16 && launch_nint_gemm(w->nint, x, m, y, y_dtype, w->device, stream)) return;
            const int mb = nint_gemv_max_batch(w->nint, w->device);
            if (mb == 0) fail(MFQB_ERR_UNSUPPORTED, "k=%lld is too long for the shared-memory staging of the GEMV", (long long)k);
            for (int m0 = 0; m0 < m; m0 += mb) {
                const int mm = std::min(mb, m - m0);
                launch_nint_gemv(w->nint, static_cast<const char*>(x) + (size_t)m0 * k * 2, mm,
                                 static_cast<char*>(y) + (size_t)m0 * n * ysz, y_dtype, (int)n, w->device, stream);
            }
        } else {
            nvq_mul_mat(*w->nvq, x, m, y, y_dtype, stream);
        }
    });
}

int mfqb_mul_mat_host(const mfqb_weight* w, const void* x_host, int m, void* y_host, int y_dtype) {
    return guarded([&] {
        if (!w || !x_host || !y_host) fail(MFQB_ERR_ARG, "mfqb_mul_mat_host: null argument");
        if (m < 1) fail(MFQB_ERR_ARG, "mfqb_mul_mat_host: m must be >= 1");
        DeviceGuard guard(w->device);
        const size_t xb = (size_t)m * w->info.k * 2, yb = (size_t)m * w->info.n * (y_dtype == MFQB_F32 ? 4 : 2);
        DevBuf dx, dy;
        dx.alloc(xb);
        dy.alloc(yb);
        cudaStream_t s = nullptr;
        MFQB_CUDA(cudaMemcpyAsync(dx.p, x_host, xb, cudaMemcpyHostToDevice, s));
        const int rc = mfqb_mul_mat(w, dx.p, m, dy.p, y_dtype, s);
        if (rc != MFQB_OK) throw Error(rc, mfqb_last_error());
        MFQB_CUDA(cudaMemcpyAsync(y_host, dy.p, yb, cudaMemcpyDeviceToHost, s));
        MFQB_CUDA(cudaStreamSynchronize(s));
    });
}

int mfqb_device_status(int device, int* status) {
    return guarded([&] {
        if (!status || device < 0 || device >= 64) fail(MFQB_ERR_ARG, "mfqb_device_status: bad argument");
        *status = gemm_device_status(device);
    });
}

int mfqb_selfcheck_layout(const char* dtype, const void* blob, uint64_t nbytes, uint64_t* mismatches) {
    return guarded([&] {
        if (!dtype || !blob || !mismatches) fail(MFQB_ERR_ARG, "mfqb_selfcheck_layout: null argument");
        const std::string d(dtype);
        if (dtype_is_nint(d)) {
            HostNint t = parse_nint(blob, nbytes);
            check_nint_supported(t);
            *mismatches = selfcheck_nint_layout(t);
        } else if (dtype_is_nvq(d)) {
            *mismatches = selfcheck_nvq_layout(parse_nvq(blob, nbytes));
        } else {
            fail(MFQB_ERR_UNSUPPORTED, "dtype '%s' is outside the packed-weight execution path", dtype);
        }
    });
}

#pragma GCC visibility pop
}  // extern "C"
