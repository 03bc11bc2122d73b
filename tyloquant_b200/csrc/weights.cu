// Dense weight handles: blob -> device layout -> decode / multiply entry points.
#include <cuda_bf16.h>

#include <algorithm>
#include <memory>
#include <mutex>
#include <utility>
#include <vector>

#include <climits>

#include "cuda_util.h"
#include "nint_gemm_tc.cuh"
#include "nint_blayout.h"
#include "nvq.h"
#include "nvq_blayout.h"

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

void* GrowOnlyScratch::get(int device, size_t bytes, cudaStream_t stream, const char* what) {
    static std::mutex mu;   // one lock for every pool: growth is rare
    std::lock_guard<std::mutex> lock(mu);
    if (device < 0 || device >= 64) fail(MFQB_ERR_ARG, "device index %d out of range", device);
    PerDevice& d = dev_[device];
    if (d.bytes >= bytes) return d.p;
    cudaStreamCaptureStatus st = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(stream, &st) != cudaSuccess) (void)cudaGetLastError();
    if (st != cudaStreamCaptureStatusNone)
        fail(MFQB_ERR_ARG,
             "%s needs %zu bytes of library scratch (it holds %zu) while the stream is being captured: "
             "run one call of this size outside the capture first",
             what, bytes, d.bytes);
    void* p = nullptr;
    const size_t want = bytes + bytes / 2;
    MFQB_CUDA(cudaMalloc(&p, want));
    MFQB_CUDA(cudaMemset(p, 0, want));   // some users keep self-resetting counters in their block: they start at zero
    d.p = p;   // the previous block stays allocated: earlier launches and captured graphs may still use it
    d.bytes = want;
    return p;
}

// ---- tcgen05 prefill GEMM: x conversion pre-pass, per-device scratch and status word -----------
__global__ void x_to_f16_kernel(const __nv_bfloat16* __restrict__ x, int m, int k, int kx, __half* __restrict__ out) {
    const size_t total = (size_t)m * kx;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const size_t r = i / kx, c = i % kx;
        // bf16 -> f16: exact for |x| in [2^-14, 65504]; larger finite magnitudes saturate to +-65504;
        // an infinity or NaN stays non-finite (NaN), so it poisons the outputs as on the integer kernels
        const float v = c < (size_t)k ? __bfloat162float(x[r * k + c]) : 0.f;
        out[i] = isfinite(v) ? __float2half_rn(fminf(fmaxf(v, -65504.f), 65504.f)) : __ushort_as_half((unsigned short)0x7E00);
    }
}

struct GemmDeviceState {
    std::mutex mu;
    GrowOnlyScratch x16;
    int* status_host[64] = {nullptr};
    int* status_dev[64] = {nullptr};
};
static GemmDeviceState g_gemm;

int* gemm_status_word(int device) {   // pinned, mapped: the host can read it without a sync
    if (!g_gemm.status_host[device]) {
        MFQB_CUDA(cudaHostAlloc((void**)&g_gemm.status_host[device], sizeof(int), cudaHostAllocMapped));
        *g_gemm.status_host[device] = 0;
        MFQB_CUDA(cudaHostGetDevicePointer((void**)&g_gemm.status_dev[device], g_gemm.status_host[device], 0));
    }
    return g_gemm.status_dev[device];
}

// Tensor map of the f16 activations [m, kx] for 64-column x bn-row boxes with the 128-byte swizzle.
// cuTensorMapEncodeTiled is looked up through the runtime, so the library links only libcudart.
static CUtensorMap make_x_map(const void* x16, int m, int kx, int bn, int xcols = 64) {
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
    const cuuint32_t box[2] = {(cuuint32_t)xcols, (cuuint32_t)std::min(bn, 256)};   // a box holds at most 256 rows; wider tiles take two loads
    const cuuint32_t elem[2] = {1u, 1u};
    const CUresult r = encode(&map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(x16), dims, strides, box, elem,
                              CU_TENSOR_MAP_INTERLEAVE_NONE, xcols == 64 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) fail(MFQB_ERR_CUDA, "cuTensorMapEncodeTiled failed with code %d", (int)r);
    return map;
}

// Returns false when this weight has no tensor-core tile kernel (the caller falls back to GEMV passes).
int* device_status_word(int device) {
    std::lock_guard<std::mutex> lock(g_gemm.mu);
    return gemm_status_word(device);
}

static bool launch_nint_gemm(const NintDevB& w, const void* x, int m, void* y, int y_dtype, int device, cudaStream_t s) {
    const GemmPlan p = plan_nint_gemm(w, m);
    if (p.bn == 0) return false;
    std::lock_guard<std::mutex> lock(g_gemm.mu);
    GemmArgs a{};
    a.w = w;
    a.m = m;
    a.kx = (w.k + 7) / 8 * 8;
    a.y = y;
    a.y_dtype = y_dtype;
    a.bn = p.bn;
    a.stages = p.stages;
    a.xstages = p.xstages;
    a.xcols = p.xcols;
    a.error = gemm_status_word(device);
    void* xb = g_gemm.x16.get(device, (size_t)m * a.kx * sizeof(__half), s, "mfqb_mul_mat (f16 copy of the activations)");
    a.x16 = static_cast<const __half*>(xb);
    const size_t total = (size_t)m * a.kx;
    x_to_f16_kernel<<<(int)std::min<size_t>((total + 255) / 256, 148 * 8), 256, 0, s>>>(static_cast<const __nv_bfloat16*>(x), m, w.k,
                                                                                      a.kx, static_cast<__half*>(xb));
    MFQB_CUDA(cudaGetLastError());
    const CUtensorMap x_map = make_x_map(xb, m, a.kx, p.bn, p.xcols);
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

// Rows of x (bf16 [rows, k]) gathered in route-plan order and converted to f16 [pairs, kx]:
// out row p = x row (pair_order[p] / div).
template <typename XT>
__global__ void x_gather_f16_kernel(const XT* __restrict__ x, const int* __restrict__ pair_order, int div, int pairs, int k, int kx,
                                    __half* __restrict__ out) {
    const size_t total = (size_t)pairs * kx;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const size_t p = i / kx, c = i % kx;
        const float v = c < (size_t)k ? (float)x[(size_t)(pair_order[p] / div) * k + c] : 0.f;
        out[i] = isfinite(v) ? __float2half_rn(fminf(fmaxf(v, -65504.f), 65504.f)) : __ushort_as_half((unsigned short)0x7E00);
    }
}

// True when the grouped tile kernel can run this cohort tensor with `bn`-pair tiles.
bool nint_gemm_grouped_supported(const NintDevB& w, int bn, int rows_per_expert) { return plan_nint_gemm_grouped(w, bn, rows_per_expert, 1).bn != 0; }

// Bytes of the gathered f16 input the grouped kernel reads.
size_t nint_gemm_grouped_x_bytes(int pairs, int k) { return (size_t)pairs * ((k + 7) / 8 * 8) * sizeof(__half); }

void launch_x_gather_f16(const void* x, bool x_f32, const int* pair_order, int div, int pairs, int k, void* x16, cudaStream_t s) {
    const int kx = (k + 7) / 8 * 8;
    const size_t total = (size_t)pairs * kx;
    const int grid = (int)std::min<size_t>((total + 255) / 256, 148 * 8);
    if (x_f32) x_gather_f16_kernel<float><<<grid, 256, 0, s>>>(static_cast<const float*>(x), pair_order, div, pairs, k, kx, static_cast<__half*>(x16));
    else x_gather_f16_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>(static_cast<const __nv_bfloat16*>(x), pair_order, div, pairs, k, kx, static_cast<__half*>(x16));
    MFQB_CUDA(cudaGetLastError());
}

// Expert matmul of one cohort on the tile kernel: x16 = launch_x_gather_f16 output for this plan.
void launch_nint_gemm_grouped(const NintDevB& w, const void* x16, int pairs, int bn, const int* expert_bounds, const int* tile_bounds,
                              const int* pair_order, const int* expert_pool, const int* expert_local, int n_experts, int pool,
                              int rb_per_expert, int rows_per_expert, int max_tiles, void* y, int y_dtype, int device, cudaStream_t s) {
    const GemmPlan p = plan_nint_gemm_grouped(w, bn, rows_per_expert, max_tiles);
    if (p.bn == 0) fail(MFQB_ERR_UNSUPPORTED, "NINT%d gs=%d has no grouped tile kernel for tiles of %d", w.bits, w.gs, bn);
    GemmArgs a{};
    {
        std::lock_guard<std::mutex> lock(g_gemm.mu);
        a.error = gemm_status_word(device);
    }
    a.w = w;
    a.m = pairs;
    a.kx = (w.k + 7) / 8 * 8;
    a.x16 = static_cast<const __half*>(x16);
    a.y = y;
    a.y_dtype = y_dtype;
    a.bn = p.bn;
    a.stages = p.stages;
    a.xstages = p.xstages;
    a.xcols = p.xcols;
    a.expert_bounds = expert_bounds;
    a.tile_bounds = tile_bounds;
    a.pair_order = pair_order;
    a.expert_pool = expert_pool;
    a.expert_local = expert_local;
    a.n_experts = n_experts;
    a.pool = pool;
    a.rb_per_expert = rb_per_expert;
    a.ldy = rows_per_expert;
    const CUtensorMap x_map = make_x_map(x16, pairs, a.kx, p.bn);
    cudaError_t e;
    switch (w.bits) {
        case 2: e = launch_nint_gemm_bits<2>(a, p, x_map, s); break;
        case 3: e = launch_nint_gemm_bits<3>(a, p, x_map, s); break;
        case 4: e = launch_nint_gemm_bits<4>(a, p, x_map, s); break;
        case 5: e = launch_nint_gemm_bits<5>(a, p, x_map, s); break;
        case 6: e = launch_nint_gemm_bits<6>(a, p, x_map, s); break;
        case 8: e = launch_nint_gemm_bits<8>(a, p, x_map, s); break;
        default: e = cudaErrorNotSupported; break;
    }
    if (e != cudaSuccess) fail(MFQB_ERR_CUDA, "NINT%d gs=%d grouped GEMM launch: %s", w.bits, w.gs, cudaGetErrorString(e));
}

int gemm_device_status(int device) {
    std::lock_guard<std::mutex> lock(g_gemm.mu);
    return g_gemm.status_host[device] ? *static_cast<volatile int*>(g_gemm.status_host[device]) : 0;
}

}  // namespace mfqb

using namespace mfqb;

namespace mfqb {
void launch_nint_bl_dequant(const NintDevB& w, void* out, int out_dtype, cudaStream_t s);
void launch_bl_gemv(const NintDevB& w, const void* x, int m, void* y, int y_dtype, int ldy, int device, cudaStream_t s, bool swiglu = false, bool glu = false);
bool nint_bl_supported(int bits, int gs);
size_t gemvs_fix_bytes(int device);
void launch_swiglu(const void* gate_up, int in_dtype, int rows, int f, void* hidden, cudaStream_t s);
void launch_bl_gemv_norm(const NintDevB& w, const float* h, const float* delta, const float* gamma, float eps, float* h_out, void* y, int y_dtype,
                         bool glu, int device, cudaStream_t s);
bool nint_bl_gemvh_supported(const NintDevB& w, int rows_per_launch);
int g_moe_f16_from_x2 = 4;   // see mfqb_tune
int g_gemm_plan_choice = 0;   // see mfqb_tune
void launch_bl_gemv_multi(const NintDevB* ws, void* const* ys, int count, const void* x, int y_dtype, int device, cudaStream_t s);
bool launch_bl_gemvs(const NintDevB& w, const void* x, int x_dtype, void* y, int y_dtype, int device, void* fix, int* error, cudaStream_t s);
}

// Which single-row kernel a plain NINT weight takes: 0 = by shape (default), 1 = always the ring
// kernel, 2 = always the streamed kernel (mfqb_tune("gemv1_kernel", v)).
static int g_gemv1_choice = 0;
static bool gemv1_use_streamed(const NintDevB& w) {
    if (g_gemv1_choice == 1) return false;
    if (g_gemv1_choice == 2) return true;
    (void)w;
    return false;   // measured on B200: the ring kernel is as fast or faster on every shape of the sweep
}

struct mfqb_weight {
    int family = 0, device = 0;
    mfqb_weight_info info{};
    NintDevB nint{};
    DevBuf items, anchors;
    DevBuf fix;          // streamed single-row kernel: partial rows of row-blocks shared by two CTAs, and their counters
    int* status = nullptr;   // the device's host-visible status word
    NvqDevicePtr nvq;
};

namespace mfqb {

void check_nint_supported(const HostNint& t) {
    const int b = t.bits;
    if (!(b == 2 || b == 3 || b == 4 || b == 5 || b == 6 || b == 8))
        fail(MFQB_ERR_UNSUPPORTED, "NINT%d is not an executable code width (2,3,4,5,6,8)", b);
    if (!nint_bl_supported(b, t.gs)) fail(MFQB_ERR_UNSUPPORTED, "NINT%d with groupsize %d is outside the runtime catalog", b, t.gs);
}

const NintDevB& weight_device_layout(const mfqb_weight* w);
int weight_device_index(const mfqb_weight* w);

static mfqb_weight* make_nint_weight(const HostNint& t, int device) {
    check_nint_supported(t);
    NintPackedB p = pack_nint_bytes(t);
    auto w = std::make_unique<mfqb_weight>();
    DeviceGuard guard(device);
    w->family = MFQB_FAMILY_NINT;
    w->device = device;
    w->items.upload(p.items.data(), p.items.size() * 4);
    w->anchors.upload(p.anchors.data(), p.anchors.size() * 4);
    w->fix.alloc(gemvs_fix_bytes(device));
    MFQB_CUDA(cudaMemset(w->fix.p, 0, w->fix.bytes));
    w->status = device_status_word(device);
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

const NintDevB& weight_device_layout(const mfqb_weight* w) { return w->family == MFQB_FAMILY_NINT ? w->nint : nvq_device_layout(*w->nvq); }
int weight_device_index(const mfqb_weight* w) { return w->device; }

}  // namespace mfqb

// prod [rows, n] float32 whose columns come in 16-wide blocks alternating gate and up -> y [rows, n / 2] = up * silu(gate)
__global__ void glu_blocks_kernel(const float* __restrict__ prod, int rows, int n, void* __restrict__ y, int y_dtype) {
    const int half = n >> 1;
    const size_t total = (size_t)rows * half;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const size_t r = i / half;
        const int j = (int)(i % half), blk = j >> 4, lane = j & 15;
        const float g = prod[r * n + blk * 32 + lane], u = prod[r * n + blk * 32 + 16 + lane];
        const float v = u * g / (1.0f + expf(-g));
        if (y_dtype == MFQB_F32) static_cast<float*>(y)[i] = v;
        else static_cast<__nv_bfloat16*>(y)[i] = __float2bfloat16_rn(v);
    }
}

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

int mfqb_weight_clone(const mfqb_weight* src, mfqb_weight** out) {
    return guarded([&] {
        if (!src || !out) fail(MFQB_ERR_ARG, "mfqb_weight_clone: null argument");
        if (src->family != MFQB_FAMILY_NINT) fail(MFQB_ERR_UNSUPPORTED, "mfqb_weight_clone: only scalar-quantised (NINT) weights");
        DeviceGuard guard(src->device);
        auto w = std::make_unique<mfqb_weight>();
        w->family = src->family;
        w->device = src->device;
        w->info = src->info;
        w->items.alloc(src->items.bytes);
        w->anchors.alloc(src->anchors.bytes);
        MFQB_CUDA(cudaMemcpy(w->items.p, src->items.p, src->items.bytes, cudaMemcpyDeviceToDevice));
        MFQB_CUDA(cudaMemcpy(w->anchors.p, src->anchors.p, src->anchors.bytes, cudaMemcpyDeviceToDevice));
        w->fix.alloc(src->fix.bytes);
        MFQB_CUDA(cudaMemset(w->fix.p, 0, w->fix.bytes));
        w->status = src->status;
        w->nint = src->nint;
        w->nint.items = static_cast<const uint32_t*>(w->items.p);
        w->nint.anchors = static_cast<const uint32_t*>(w->anchors.p);
        *out = w.release();
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
        if (w->family == MFQB_FAMILY_NINT) launch_nint_bl_dequant(w->nint, out, out_dtype, stream);
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
            if (m == 1 && gemv1_use_streamed(w->nint) &&
                launch_bl_gemvs(w->nint, x, MFQB_BF16, y, y_dtype, w->device, w->fix.p, w->status, stream))
                return;
            const int per_launch = nint_bl_gemvh_supported(w->nint, 16) ? 16 : 8;   // batch rows one GEMV launch covers
            for (int m0 = 0; m0 < m; m0 += per_launch) {
                const int mm = std::min(per_launch, m - m0);
                launch_bl_gemv(w->nint, static_cast<const char*>(x) + (size_t)m0 * k * 2, mm,
                                    static_cast<char*>(y) + (size_t)m0 * n * ysz, y_dtype, (int)n, w->device, stream);
            }
        } else {
            nvq_mul_mat(*w->nvq, x, m, y, y_dtype, stream);
        }
    });
}

int mfqb_mul_mat_swiglu(const mfqb_weight* w, const void* gate_up, int m, void* y, int y_dtype, mfqb_stream_t stream) {
    return guarded([&] {
        if (!w || !gate_up || !y) fail(MFQB_ERR_ARG, "mfqb_mul_mat_swiglu: null argument");
        if (m < 1) fail(MFQB_ERR_ARG, "mfqb_mul_mat_swiglu: m must be >= 1, got %d", m);
        if (y_dtype != MFQB_F32 && y_dtype != MFQB_BF16) fail(MFQB_ERR_ARG, "mfqb_mul_mat_swiglu: bad output dtype");
        if (w->info.k > INT_MAX) fail(MFQB_ERR_ARG, "mfqb_mul_mat_swiglu: row length out of range");
        DeviceGuard guard(w->device);
        if (m == 1 && w->family == MFQB_FAMILY_NINT) {   // activation computed as the down projection loads its row
            launch_bl_gemv(w->nint, gate_up, 1, y, y_dtype, (int)w->info.n, w->device, stream, true);
            return;
        }
        static GrowOnlyScratch pool;
        void* act = pool.get(w->device, (size_t)m * w->info.k * 2, stream, "mfqb_mul_mat_swiglu (activation rows)");
        launch_swiglu(gate_up, MFQB_F32, m, (int)w->info.k, act, stream);
        const int rc = mfqb_mul_mat(w, act, m, y, y_dtype, stream);
        if (rc != MFQB_OK) throw Error(rc, mfqb_last_error());
    });
}

int mfqb_mul_mat_rmsnorm(const mfqb_weight* w, const float* h, const float* delta, const float* gamma, float eps, float* h_out, void* y,
                         int y_dtype, int gated, mfqb_stream_t stream) {
    return guarded([&] {
        if (!w || !h || !gamma || !y) fail(MFQB_ERR_ARG, "mfqb_mul_mat_rmsnorm: null argument");
        if (y_dtype != MFQB_F32 && y_dtype != MFQB_BF16) fail(MFQB_ERR_ARG, "mfqb_mul_mat_rmsnorm: bad output dtype");
        if (h_out == h) fail(MFQB_ERR_ARG, "mfqb_mul_mat_rmsnorm: h_out must not be h (other CTAs still read h)");
        if (w->family != MFQB_FAMILY_NINT || w->nint.table) fail(MFQB_ERR_UNSUPPORTED, "mfqb_mul_mat_rmsnorm: scalar-quantised (NINT) weights only");
        DeviceGuard guard(w->device);
        launch_bl_gemv_norm(w->nint, h, delta, gamma, eps, h_out, y, y_dtype, gated != 0, w->device, stream);
    });
}

int mfqb_mul_mat_glu(const mfqb_weight* w, const void* x, int m, void* y, int y_dtype, mfqb_stream_t stream) {
    return guarded([&] {
        if (!w || !x || !y) fail(MFQB_ERR_ARG, "mfqb_mul_mat_glu: null argument");
        if (m < 1) fail(MFQB_ERR_ARG, "mfqb_mul_mat_glu: m must be >= 1, got %d", m);
        if (y_dtype != MFQB_F32 && y_dtype != MFQB_BF16) fail(MFQB_ERR_ARG, "mfqb_mul_mat_glu: bad output dtype");
        if (w->info.n % 32) fail(MFQB_ERR_ARG, "mfqb_mul_mat_glu: the weight needs whole (gate, up) pairs of 16-row blocks, n = %lld", (long long)w->info.n);
        DeviceGuard guard(w->device);
        if (m == 1 && w->family == MFQB_FAMILY_NINT) {   // activation applied where the kernel writes its rows
            launch_bl_gemv(w->nint, x, 1, y, y_dtype, (int)w->info.n, w->device, stream, false, true);
            return;
        }
        static GrowOnlyScratch pool;
        float* prod = static_cast<float*>(pool.get(w->device, (size_t)m * w->info.n * 4, stream, "mfqb_mul_mat_glu (gate and up products)"));
        const int rc = mfqb_mul_mat(w, x, m, prod, MFQB_F32, stream);
        if (rc != MFQB_OK) throw Error(rc, mfqb_last_error());
        const size_t total = (size_t)m * (w->info.n / 2);
        glu_blocks_kernel<<<(unsigned)std::min<size_t>((total + 255) / 256, 148 * 8), 256, 0, stream>>>(prod, m, (int)w->info.n, y, y_dtype);
        MFQB_CUDA(cudaGetLastError());
    });
}

int mfqb_mul_mat_multi(const mfqb_weight* const* ws, int count, const void* x, void* const* ys, int y_dtype, mfqb_stream_t stream) {
    return guarded([&] {
        if (!ws || !x || !ys) fail(MFQB_ERR_ARG, "mfqb_mul_mat_multi: null argument");
        if (count < 1 || count > 8) fail(MFQB_ERR_ARG, "mfqb_mul_mat_multi: 1 to 8 weights per call, got %d", count);
        if (y_dtype != MFQB_F32 && y_dtype != MFQB_BF16) fail(MFQB_ERR_ARG, "mfqb_mul_mat_multi: bad output dtype");
        NintDevB devs[8];
        for (int i = 0; i < count; ++i) {
            if (!ws[i] || !ys[i]) fail(MFQB_ERR_ARG, "mfqb_mul_mat_multi: null weight or output");
            if (ws[i]->family != MFQB_FAMILY_NINT) fail(MFQB_ERR_UNSUPPORTED, "mfqb_mul_mat_multi: scalar-quantised (NINT) weights only");
            if (ws[i]->device != ws[0]->device) fail(MFQB_ERR_ARG, "mfqb_mul_mat_multi: weights live on different devices");
            devs[i] = ws[i]->nint;
        }
        DeviceGuard guard(ws[0]->device);
        launch_bl_gemv_multi(devs, ys, count, x, y_dtype, ws[0]->device, stream);
    });
}

// Copies `words` 32-bit words (activations in mapped pinned host memory -> device staging).
__global__ void host_to_device_words_kernel(const uint32_t* __restrict__ src, uint32_t* __restrict__ dst, size_t words) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < words; i += (size_t)gridDim.x * blockDim.x) dst[i] = src[i];
}

// The same for up to 32 buffers in one launch (blockIdx.y picks the buffer): one trip over PCIe for all of them.
struct HostGatherTable {
    const uint32_t* src[32];
    uint32_t* dst[32];
    unsigned words[32];
};
__global__ void host_gather_words_kernel(const __grid_constant__ HostGatherTable t) {
    const uint32_t* src = t.src[blockIdx.y];
    uint32_t* dst = t.dst[blockIdx.y];
    const unsigned words = t.words[blockIdx.y];
    for (unsigned i = blockIdx.x * blockDim.x + threadIdx.x; i < words; i += gridDim.x * blockDim.x) dst[i] = src[i];
}

// Device staging of the host-buffer entry point: per device one stream and two buffers that grow on
// demand and are then reused, so a call costs two copies, the kernel and one synchronisation.
namespace {
struct HostCallState {
    std::mutex mu[64];
    cudaStream_t stream[64] = {nullptr};
    cudaEvent_t done[64] = {nullptr};
    DevBuf x[64], y[64];
};
HostCallState g_host_call;
}  // namespace

// Host-buffer products: `count` weights of one device, each with its own x and y in host memory.
// Everything is enqueued on the device's staging stream and the call waits once, at the end.
static void mul_mat_host_impl(const mfqb_weight* const* ws, int count, const void* const* xs, int m, void* const* ys, int y_dtype) {
    const mfqb_weight* w0 = ws[0];
    if (w0->device < 0 || w0->device >= 64) fail(MFQB_ERR_ARG, "device index %d out of range", w0->device);
    const int device = w0->device;
    DeviceGuard guard(device);
    const size_t ysz = y_dtype == MFQB_F32 ? 4 : 2;
    size_t x_total = 0, y_total = 0;
    for (int i = 0; i < count; ++i) {
        if (!ws[i] || !xs[i] || !ys[i]) fail(MFQB_ERR_ARG, "mfqb_mul_mat_host: null argument");
        if (ws[i]->device != device) fail(MFQB_ERR_ARG, "mfqb_mul_mat_host_multi: weights live on different devices");
        x_total += ((size_t)m * ws[i]->info.k * 2 + 255) / 256 * 256;
        y_total += ((size_t)m * ws[i]->info.n * ysz + 255) / 256 * 256;
    }
    std::lock_guard<std::mutex> lock(g_host_call.mu[device]);   // per device: calls on different GPUs do not serialise
    cudaStream_t& s = g_host_call.stream[device];
    if (!s) MFQB_CUDA(cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking));
    cudaEvent_t& ev = g_host_call.done[device];
    if (!ev) MFQB_CUDA(cudaEventCreateWithFlags(&ev, cudaEventDisableTiming));
    DevBuf& dx = g_host_call.x[device];
    DevBuf& dy = g_host_call.y[device];
    if (dx.bytes < x_total) dx.alloc(x_total + x_total / 2);   // nothing of this stream is in flight between calls
    size_t x_off = 0, y_off = 0;
    bool any_copy_back = false;
    // Pinned, mapped host buffers (cudaHostAlloc / cudaHostRegister, which is what a caller that
    // cares about latency passes): a small kernel pulls x over PCIe into the staging buffer and the
    // product kernel writes y straight into host memory -- no copy-engine round trips.  Pageable
    // buffers take the two cudaMemcpyAsync.
    std::vector<std::pair<size_t, int>> copy_back;   // (offset in dy, index)
    // First every activation buffer is staged (the mapped ones 32 per launch), then the products run
    // back to back: consecutive product kernels overlap through programmatic dependent launch, which
    // a staging kernel between them would break.
    std::vector<char*> xd(count);
    std::vector<void*> yd(count);
    HostGatherTable table{};
    int pending = 0;
    unsigned max_words = 0;
    auto flush = [&]() {
        if (!pending) return;
        const dim3 grid(std::max(1u, std::min((max_words + 255) / 256, 16u)), (unsigned)pending);
        host_gather_words_kernel<<<grid, 256, 0, s>>>(table);
        MFQB_CUDA(cudaGetLastError());
        pending = 0;
        max_words = 0;
    };
    for (int i = 0; i < count; ++i) {
        const size_t xb = (size_t)m * ws[i]->info.k * 2, yb = (size_t)m * ws[i]->info.n * ysz;
        void *x_map = nullptr, *y_map = nullptr;
        const bool mapped = (xb % 4 == 0) && xb / 4 <= 0xFFFFFFFFull && (reinterpret_cast<uintptr_t>(xs[i]) % 4 == 0) &&
                            cudaHostGetDevicePointer(&x_map, const_cast<void*>(xs[i]), 0) == cudaSuccess &&
                            cudaHostGetDevicePointer(&y_map, ys[i], 0) == cudaSuccess;
        if (!mapped) (void)cudaGetLastError();   // not an error: the buffers are simply pageable
        if (i > 0 && xs[i] == xs[i - 1] && ws[i]->info.k == ws[i - 1]->info.k) {   // the same host rows as the previous product: staged once
            xd[i] = xd[i - 1];
            if (!mapped) {
                if (!any_copy_back && dy.bytes < y_total) dy.alloc(y_total + y_total / 2);
                any_copy_back = true;
                copy_back.emplace_back(y_off, i);
            }
            yd[i] = mapped ? y_map : static_cast<void*>(static_cast<char*>(dy.p) + y_off);
            y_off += (yb + 255) / 256 * 256;
            continue;
        }
        xd[i] = static_cast<char*>(dx.p) + x_off;
        if (mapped) {
            table.src[pending] = static_cast<const uint32_t*>(x_map);
            table.dst[pending] = reinterpret_cast<uint32_t*>(xd[i]);
            table.words[pending] = (unsigned)(xb / 4);
            max_words = std::max(max_words, (unsigned)(xb / 4));
            if (++pending == 32) flush();
        } else {
            MFQB_CUDA(cudaMemcpyAsync(xd[i], xs[i], xb, cudaMemcpyHostToDevice, s));
            if (!any_copy_back && dy.bytes < y_total) dy.alloc(y_total + y_total / 2);
            any_copy_back = true;
            copy_back.emplace_back(y_off, i);
        }
        yd[i] = mapped ? y_map : static_cast<void*>(static_cast<char*>(dy.p) + y_off);
        x_off += (xb + 255) / 256 * 256;
        y_off += (yb + 255) / 256 * 256;
    }
    flush();
    // consecutive single-row products of one shape class on the same activations (q, k, v of a block) share a launch
    auto same_class = [](const mfqb_weight* a, const mfqb_weight* b) {
        return a->family == MFQB_FAMILY_NINT && b->family == MFQB_FAMILY_NINT && !a->nint.table && !b->nint.table && a->nint.bits == b->nint.bits &&
               a->nint.gs == b->nint.gs && a->nint.k == b->nint.k && a->nint.rec_words == b->nint.rec_words;
    };
    for (int i = 0; i < count;) {
        int run = 1;
        if (m == 1)
            while (i + run < count && run < 8 && xs[i + run] == xs[i] && same_class(ws[i], ws[i + run])) ++run;
        const int rc = run > 1 ? mfqb_mul_mat_multi(ws + i, run, xd[i], yd.data() + i, y_dtype, s) : mfqb_mul_mat(ws[i], xd[i], m, yd[i], y_dtype, s);
        if (rc != MFQB_OK) throw Error(rc, mfqb_last_error());
        i += run;
    }
    for (const auto& cb : copy_back)
        MFQB_CUDA(cudaMemcpyAsync(ys[cb.second], static_cast<char*>(dy.p) + cb.first, (size_t)m * ws[cb.second]->info.n * ysz,
                                  cudaMemcpyDeviceToHost, s));
    // wait by polling an event: the answer comes back a few microseconds sooner than through a blocking synchronise
    MFQB_CUDA(cudaEventRecord(ev, s));
    for (;;) {
        const cudaError_t q = cudaEventQuery(ev);
        if (q == cudaSuccess) break;
        if (q != cudaErrorNotReady) MFQB_CUDA(q);
    }
}

int mfqb_mul_mat_host(const mfqb_weight* w, const void* x_host, int m, void* y_host, int y_dtype) {
    return guarded([&] {
        if (!w || !x_host || !y_host) fail(MFQB_ERR_ARG, "mfqb_mul_mat_host: null argument");
        if (m < 1) fail(MFQB_ERR_ARG, "mfqb_mul_mat_host: m must be >= 1");
        mul_mat_host_impl(&w, 1, &x_host, m, &y_host, y_dtype);
    });
}

int mfqb_mul_mat_host_multi(const mfqb_weight* const* ws, int count, const void* const* xs_host, int m, void* const* ys_host, int y_dtype) {
    return guarded([&] {
        if (!ws || !xs_host || !ys_host) fail(MFQB_ERR_ARG, "mfqb_mul_mat_host_multi: null argument");
        if (count < 1 || m < 1) fail(MFQB_ERR_ARG, "mfqb_mul_mat_host_multi: count and m must be >= 1");
        mul_mat_host_impl(ws, count, xs_host, m, ys_host, y_dtype);
    });
}

int mfqb_tune(const char* key, int value) {
    return guarded([&] {
        if (!key) fail(MFQB_ERR_ARG, "mfqb_tune: null key");
        if (std::string(key) == "gemv1_kernel" && value >= 0 && value <= 2) g_gemv1_choice = value;
        else if (std::string(key) == "moe_f16_tiles_from_x2" && value >= 2 && value <= 1000000) g_moe_f16_from_x2 = value;
        else if (std::string(key) == "gemm_plan" && value >= 0 && value <= 1) g_gemm_plan_choice = value;
        else fail(MFQB_ERR_ARG, "mfqb_tune: unknown key '%s' or value %d out of range", key, value);
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
            *mismatches = selfcheck_nint_bytes(t);
        } else if (dtype_is_nvq(d)) {
            *mismatches = selfcheck_nvq_bytes(parse_nvq(blob, nbytes));
        } else {
            fail(MFQB_ERR_UNSUPPORTED, "dtype '%s' is outside the packed-weight execution path", dtype);
        }
    });
}

#pragma GCC visibility pop
}  // extern "C"
