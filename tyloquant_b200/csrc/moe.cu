// Expert-wise mixed-precision weights (NINTM) on the device and the routed expert matmul.
//
// Every precision cohort of the record becomes one NINT device tensor whose rows are the held
// experts of the cohort, each padded to whole 16-row blocks.  A routed matmul launches the
// single-row kernel once per cohort over (row splits, pairs) CTAs (larger batches: the batched
// kernel over route-plan tiles of 8 pairs of one expert); a CTA looks its pair's expert
// up in two small tables (cohort of the expert, position inside the cohort) and returns when
// the expert belongs to another cohort or is not held by this handle (expert-parallel shard).
#include <cuda_bf16.h>

#include <algorithm>
#include <climits>
#include <memory>
#include <mutex>

#include "cuda_util.h"
#include "nint_gemv1_bl.cuh"

namespace mfqb {
void launch_swiglu(const void* gate_up, int in_dtype, int rows, int f, void* hidden, cudaStream_t s);
void launch_swiglu_f32(const float* gate_up, int rows, int f, float* hidden, cudaStream_t s);
int moe_hetero_gemv1_splits(int rb_per_expert, int pairs, int device);
bool moe_hetero_supported(const NintDevB* pools, const int* held, int npools);
void launch_weighted_reduce(const void* src, int in_dtype, const float* weights, int tokens, int routes, int h, void* y, int y_dtype,
                            cudaStream_t s);

void launch_route_plan(const int32_t* ids, int pairs, int experts, int tile_m, int32_t* expert_bounds, int32_t* tile_bounds,
                       int32_t* pair_order, cudaStream_t stream);

// Device buffers of a route plan: expert_bounds [E+1], tile_bounds [E+1], pair_order [pairs].
struct PlanBufs {
    int32_t *expert_bounds, *tile_bounds, *pair_order;
    static size_t bytes(int experts, size_t pairs) { return ((2 * ((size_t)experts + 1) + pairs) * 4 + 255) / 256 * 256; }
    static PlanBufs carve(void* p, int experts) {
        int32_t* b = static_cast<int32_t*>(p);
        return PlanBufs{b, b + experts + 1, b + 2 * (experts + 1)};
    }
};

void launch_nint_bl_dequant(const NintDevB& w, void* out, int out_dtype, cudaStream_t s);
void launch_nint_bl_gemv_routed(GemvArgsB a, int pairs, int device, cudaStream_t s);
void launch_nint_bl_gemv_tiles(GemvArgsB a, int tile_m, int max_tiles, int device, cudaStream_t s);
void check_nint_supported(const HostNint& t);
int nint_bl_max_passes(const NintDevB& w);
bool nint_gemm_grouped_supported(const NintDevB& w, int bn, int rows_per_expert);
size_t nint_gemm_grouped_x_bytes(int pairs, int k);
void launch_x_gather_f16(const void* x, bool x_f32, const int* pair_order, int div, int pairs, int k, void* x16, cudaStream_t s);
void launch_nint_gemm_grouped(const NintDevB& w, const void* x16, int pairs, int bn, const int* expert_bounds, const int* tile_bounds,
                              const int* pair_order, const int* expert_pool, const int* expert_local, int n_experts, int pool,
                              int rb_per_expert, int rows_per_expert, int max_tiles, void* y, int y_dtype, int device, cudaStream_t s);
bool moe_hetero_tilesh_supported(const NintDevB* pools, const int* held, int npools);
bool launch_moe_hetero_tilesh(GemvArgsB base, const NintDevB* pools, const int* held, int npools, int tile_m, int max_tiles, int device, cudaStream_t s);
// Twice the pairs per expert from which the f16 tile kernel is used (mfqb_tune "moe_f16_tiles_from_x2"); defined with mfqb_tune.
extern int g_moe_f16_from_x2;
size_t nint_bl_frag_tile_units(const NintDevB& w, int nt);
size_t x_frags_bytes(int in_rows, int tiles, size_t tile_units);
void launch_x_frags(XFragArgs fa, int in_rows, int tiles, int max_nchunks, void* buf, const uint2** xf, const float** down, cudaStream_t s);
bool launch_moe_hetero_tiles(GemvArgsB base, const NintDevB* pools, const int* held, const uint2* const* xq, const float2* const* gtab,
                             int npools, int tile_m, int max_tiles, int device, cudaStream_t s);
bool launch_moe_hetero_gemv1(GemvArgsB base, const NintDevB* pools, const int* held, int npools, int pairs, int device, cudaStream_t s);
size_t nint_bl_planes_bytes(const NintDevB& w, int rows);
void launch_x_planes(const NintDevB& w, const void* x, int rows, void* planes, const uint2** xq_g, const float2** gtab_g, cudaStream_t s,
                     bool x_f32);

struct MoePool {
    NintDevB d{};
    DevBuf items, anchors;
    int held = 0;   // experts of this cohort held here
};

// Rows of the listed experts (positions inside the cohort tensor), each padded with all-zero
// rows to `padded` rows.
static HostNint gather_experts(const HostNint& t, const std::vector<int>& local, int64_t ope, int64_t padded) {
    HostNint r;
    r.bits = t.bits;
    r.sub_bits = t.sub_bits;
    r.gs = t.gs;
    r.k = t.k;
    r.ng = t.ng;
    r.n = (int64_t)local.size() * padded;
    r.ns.assign(r.n, 0);
    r.nm.assign(r.n, 0);
    r.ss.assign((size_t)r.n * t.ng, 0);
    r.sm.assign((size_t)r.n * t.ng, 0);
    r.q.assign((size_t)r.n * t.ng * t.gs, 0);
    for (size_t i = 0; i < local.size(); ++i) {
        const int64_t src = (int64_t)local[i] * ope, dst = (int64_t)i * padded;
        std::copy(t.ns.begin() + src, t.ns.begin() + src + ope, r.ns.begin() + dst);
        std::copy(t.nm.begin() + src, t.nm.begin() + src + ope, r.nm.begin() + dst);
        std::copy(t.ss.begin() + src * t.ng, t.ss.begin() + (src + ope) * t.ng, r.ss.begin() + dst * t.ng);
        std::copy(t.sm.begin() + src * t.ng, t.sm.begin() + (src + ope) * t.ng, r.sm.begin() + dst * t.ng);
        std::copy(t.q.begin() + src * t.ng * t.gs, t.q.begin() + (src + ope) * t.ng * t.gs, r.q.begin() + dst * t.ng * t.gs);
    }
    return r;
}

// Per-device scratch for the FFN intermediates (slot 0) and for a stand-alone routed matmul's plan
// and planes (slot 1): grow-only, see GrowOnlyScratch.
static void* scratch_get(int device, size_t bytes, cudaStream_t stream, int slot = 0) {
    static GrowOnlyScratch pools[2];
    return pools[slot].get(device, bytes, stream, slot ? "mfqb_mul_mat_id (route plan and activation planes)" : "mfqb_moe_ffn (intermediates)");
}

}  // namespace mfqb

using namespace mfqb;

struct mfqb_moe_weight {
    mfqb_moe_info info{};
    std::vector<std::unique_ptr<MoePool>> pools;
    std::vector<int> expert_pool, expert_local;          // host copies
    std::vector<uint64_t> expert_bytes;
    DevBuf d_expert_pool, d_expert_local;
    int padded = 0;                                       // rows per expert on the device (multiple of 16)
};

static uint64_t expert_payload_bytes(const HostNint& t, int64_t ope) {
    // share of the cohort's file streams: anchors + sub-scales + sub-mins + codes of `ope` rows
    const uint64_t per_row_bits = 32ull + 2ull * t.ng * t.sub_bits + (uint64_t)t.ng * t.gs * t.bits;
    return (per_row_bits * (uint64_t)ope + 7) / 8;
}

extern "C" {
#pragma GCC visibility push(default)

int mfqb_nintm_from_blob(const void* blob, uint64_t nbytes, int expert_begin, int expert_end, int device, mfqb_moe_weight** out) {
    return guarded([&] {
        if (!blob || !out) fail(MFQB_ERR_ARG, "mfqb_nintm_from_blob: null argument");
        HostNintm t = parse_nintm(blob, nbytes);
        if (expert_end < 0) expert_end = (int)t.n_experts;
        if (expert_begin < 0 || expert_begin >= expert_end || expert_end > t.n_experts)
            fail(MFQB_ERR_ARG, "expert range [%d, %d) is outside [0, %lld)", expert_begin, expert_end, (long long)t.n_experts);
        if (t.pools.size() > 16) fail(MFQB_ERR_UNSUPPORTED, "more than 16 precision cohorts in one NINTM record");
        auto w = std::make_unique<mfqb_moe_weight>();
        DeviceGuard guard(device);
        const int64_t ope = t.out_per_expert;
        w->padded = (int)((ope + 15) / 16 * 16);
        w->expert_pool.assign((size_t)t.n_experts, -1);
        w->expert_local.assign((size_t)t.n_experts, 0);
        w->expert_bytes.assign((size_t)t.n_experts, 0);
        uint64_t payload = 0, dev_bytes = 0;
        for (auto& hp : t.pools) {
            check_nint_supported(hp.tensor);
            std::vector<int> local;
            const int pool_index = (int)w->pools.size();
            for (size_t i = 0; i < hp.expert_ids.size(); ++i) {
                const int e = hp.expert_ids[i];
                if (e < expert_begin || e >= expert_end) continue;
                w->expert_pool[e] = pool_index;
                w->expert_local[e] = (int)local.size();
                w->expert_bytes[e] = expert_payload_bytes(hp.tensor, ope);
                payload += w->expert_bytes[e];
                local.push_back((int)i);
            }
            auto pool = std::make_unique<MoePool>();
            pool->held = (int)local.size();
            if (!local.empty()) {
                NintPackedB p = pack_nint_bytes(gather_experts(hp.tensor, local, ope, w->padded));
                pool->items.upload(p.items.data(), p.items.size() * 4);
                pool->anchors.upload(p.anchors.data(), p.anchors.size() * 4);
                pool->d = p.d;
                pool->d.items = static_cast<const uint32_t*>(pool->items.p);
                pool->d.anchors = static_cast<const uint32_t*>(pool->anchors.p);
                dev_bytes += pool->items.bytes + pool->anchors.bytes;
            }
            w->pools.push_back(std::move(pool));
        }
        w->d_expert_pool.upload(w->expert_pool.data(), w->expert_pool.size() * 4);
        w->d_expert_local.upload(w->expert_local.data(), w->expert_local.size() * 4);
        mfqb_moe_info& i = w->info;
        i.n_experts = (int)t.n_experts;
        i.out_per_expert = (int)ope;
        i.k = (int)t.k;
        i.expert_begin = expert_begin;
        i.expert_end = expert_end;
        i.n_pools = (int)w->pools.size();
        i.device = device;
        i.payload_bytes = payload;
        i.device_bytes = dev_bytes + w->d_expert_pool.bytes + w->d_expert_local.bytes;
        *out = w.release();
    });
}

int mfqb_moe_info_get(const mfqb_moe_weight* w, mfqb_moe_info* info) {
    return guarded([&] {
        if (!w || !info) fail(MFQB_ERR_ARG, "mfqb_moe_info_get: null argument");
        *info = w->info;
    });
}

int mfqb_moe_expert_bytes(const mfqb_moe_weight* w, int expert, uint64_t* payload_bytes) {
    return guarded([&] {
        if (!w || !payload_bytes || expert < 0 || expert >= w->info.n_experts) fail(MFQB_ERR_ARG, "mfqb_moe_expert_bytes: bad argument");
        *payload_bytes = w->expert_bytes[expert];
    });
}

int mfqb_moe_weight_free(mfqb_moe_weight* w) {
    return guarded([&] {
        if (!w) return;
        DeviceGuard guard(w->info.device);
        delete w;
    });
}

int mfqb_moe_dequant_expert(const mfqb_moe_weight* w, int expert, void* out, int out_dtype, mfqb_stream_t stream) {
    return guarded([&] {
        if (!w || !out) fail(MFQB_ERR_ARG, "mfqb_moe_dequant_expert: null argument");
        if (out_dtype != MFQB_F32 && out_dtype != MFQB_BF16) fail(MFQB_ERR_ARG, "mfqb_moe_dequant_expert: bad output dtype");
        if (expert < 0 || expert >= w->info.n_experts || w->expert_pool[expert] < 0)
            fail(MFQB_ERR_ARG, "expert %d is not held by this handle", expert);
        DeviceGuard guard(w->info.device);
        const MoePool& pool = *w->pools[w->expert_pool[expert]];
        NintDevB view = pool.d;   // the expert's row-blocks as a tensor of its own
        const int rb0 = w->expert_local[expert] * (w->padded / 16);
        view.items += (size_t)rb0 * view.nchunks * view.rec_words;
        view.anchors += (size_t)rb0 * 16;
        view.n = w->info.out_per_expert;
        view.nrb = w->padded / 16;
        launch_nint_bl_dequant(view, out, out_dtype, stream);
    });
}

// Pairs per route-plan tile (2, 4 or 8, by the average number of pairs an expert sees), or
// 0: fewer pairs than experts, every pair runs as a single-row problem of its own.
// True when the f16 tile kernel can serve every held cohort of this record.
static bool moe_f16_tiles_ok(const mfqb_moe_weight* w) {
    NintDevB devs[16];
    int held[16];
    if (w->pools.size() > 16) return false;
    for (size_t pi = 0; pi < w->pools.size(); ++pi) {
        devs[pi] = w->pools[pi]->d;
        held[pi] = w->pools[pi]->held;
    }
    return moe_hetero_tilesh_supported(devs, held, (int)w->pools.size());
}
// 8-byte units per tile of the fragment-ordered input rows (the largest among the held cohorts) and the most chunks a row has.
static size_t moe_frag_tile_units(const mfqb_moe_weight* w, int nt) {
    size_t units = 0;
    for (const auto& pool : w->pools)
        if (pool->held) units = std::max(units, nint_bl_frag_tile_units(pool->d, nt));
    return units;
}
static int moe_max_nchunks(const mfqb_moe_weight* w) {
    int n = 0;
    for (const auto& pool : w->pools)
        if (pool->held) n = std::max(n, pool->d.nchunks);
    return n;
}
// Upper bound on the route plan's tiles for `pairs` pairs in tiles of tile_m.
static int moe_max_tiles(const mfqb_moe_weight* w, int pairs, int tile_m) { return pairs / tile_m + std::min(pairs, w->info.n_experts); }


static int moe_tile_m(const mfqb_moe_weight* w, int pairs) {
    const int e = w->info.n_experts;
    if (pairs < e) return 0;
    int cap = 8;   // cohorts with wide records fit fewer batch rows per CTA
    for (const auto& pool : w->pools)
        if (pool->held) cap = std::min(cap, 2 * nint_bl_max_passes(pool->d));
    // from about three pairs per expert the f16 tile kernel (tiles of 8, then 16 pairs: an expert's weights are
    // decoded once per tile) is cheaper than the integer passes over tiles of 2 or 4
    if (2 * (long long)pairs >= (long long)mfqb::g_moe_f16_from_x2 * e && moe_f16_tiles_ok(w)) return pairs >= 10 * e ? 16 : 8;
    // measured on the 128-expert top-8 layer: tiles of four win from two to about twenty pairs per expert
    return std::min(cap, 2 * pairs <= 3 * e ? 2 : (pairs <= 24 * e ? 4 : 8));
}

// Token tile of the tensor-core tile kernel for large batches (the route plan is then built with
// this tile size), or 0 to stay on the integer kernels.  Measured on the 128-expert top-8 layer:
// from about two dozen pairs per expert one f16 decode of an expert's weights per tile beats the
// batched integer passes over them (the tile kernel's time hardly depends on the batch).
static int moe_gemm_bn(const mfqb_moe_weight* w, int pairs) {
    const int e = w->info.n_experts;
    if (pairs < 24 * e) return 0;
    int bn = 32;
    while (bn < 256 && 4 * bn < 5 * (pairs / e)) bn *= 2;   // room for experts that draw more than the average
    for (const auto& pool : w->pools)
        if (pool->held && !nint_gemm_grouped_supported(pool->d, bn, w->info.out_per_expert)) return 0;
    return bn;
}

// Bytes of quantised activation planes the tile path needs for `rows` input rows: one set per
// distinct group size among the held cohorts (cohorts of equal group size share theirs).
static size_t moe_planes_bytes(const mfqb_moe_weight* w, int rows, int pairs, int tile_m) {
    // the f16 tile kernel's fragment-ordered input rows share the space
    const size_t f16_rows = (tile_m == 8 || tile_m == 16)
                                ? (x_frags_bytes(rows, moe_max_tiles(w, pairs, tile_m), moe_frag_tile_units(w, tile_m / 8)) + 255) / 256 * 256
                                : 0;
    size_t total = 0;
    for (size_t pi = 0; pi < w->pools.size(); ++pi) {
        if (!w->pools[pi]->held) continue;
        bool seen = false;
        for (size_t pj = 0; pj < pi; ++pj) seen = seen || (w->pools[pj]->held && w->pools[pj]->d.gs == w->pools[pi]->d.gs);
        if (!seen) total += (nint_bl_planes_bytes(w->pools[pi]->d, rows) + 255) / 256 * 256;
    }
    return std::max(total, f16_rows);
}

// plan == nullptr: one single-row problem per pair.  Otherwise the batched kernel runs over the
// plan's tiles (the plan must have been built for these ids with the same tile_m) and `planes` is
// moe_planes_bytes() of device memory for the quantised input rows.
constexpr size_t kFfnCounterBytes = 64 * 1024;   // route-sum counters at the start of the FFN scratch: zero between calls
struct FfnLayout {
    bool gemm, tiles, fused_tail;
    int tile_m;
    size_t o_gu, o_hid, o_dn, o_plan, o_planes, b_pgu, total;
};

// x_mode: 0 = x is bf16; 1 = float32; 2 = float32 gate|up products [pairs, 2k], the SwiGLU activation is
// formed while loading (single-row path only).  `tail` (single-row path only): the product ends the
// FFN -- see GemvArgsB::route_w.
struct FfnTail {
    const float* route_w;
    float* pair_out;
    unsigned* token_count;
    void* y;
    int y_dtype;
};
static void mul_mat_id_impl(const mfqb_moe_weight* w, const void* x, int x_per_pair, const int32_t* ids, int tokens, int routes,
                            void* out, int out_dtype, const PlanBufs* plan, int tile_m, void* planes, cudaStream_t stream, bool gemm = false,
                            int x_mode = 0, const FfnTail* tail = nullptr) {
    const int pairs = tokens * routes, ope = w->info.out_per_expert;
    const int in_rows = x_per_pair ? pairs : tokens;
    struct PlaneSet { int gs; const uint2* xq; const float2* gtab; };
    std::vector<PlaneSet> sets;
    char* planes_next = static_cast<char*>(planes);
    // Routes to experts this handle does not hold produce zeros (expert-parallel shards are
    // summed afterwards), so clear the output when the handle is partial.
    if (!tail && w->info.expert_end - w->info.expert_begin != w->info.n_experts)
        MFQB_CUDA(cudaMemsetAsync(out, 0, (size_t)pairs * ope * (out_dtype == MFQB_F32 ? 4 : 2), stream));
    if ((x_mode == 2 || tail) && plan) fail(MFQB_ERR_ARG, "mul_mat_id: the fused activation and the fused route sum belong to the single-row path");
    if (!plan && pairs <= 32768) {   // decode sizes: all cohorts in one launch when their codecs allow
        GemvArgsB a{};
        a.x = static_cast<const __nv_bfloat16*>(x);
        a.y = out;
        a.ldy = ope;
        a.y_dtype = out_dtype;
        a.route_ids = ids;
        a.expert_pool = static_cast<const int*>(w->d_expert_pool.p);
        a.expert_local = static_cast<const int*>(w->d_expert_local.p);
        a.rb_per_expert = w->padded / 16;
        a.routes = routes;
        a.x_per_pair = x_per_pair ? 1 : 0;
        a.n_experts = w->info.n_experts;
        a.x_mode = x_mode;
        if (tail) {
            a.route_w = tail->route_w;
            a.pair_out = tail->pair_out;
            a.token_count = tail->token_count;
            a.y_final = tail->y;
            a.y_final_dtype = tail->y_dtype;
        }
        NintDevB devs[16];
        int held[16];
        for (size_t pi = 0; pi < w->pools.size(); ++pi) {
            devs[pi] = w->pools[pi]->d;
            held[pi] = w->pools[pi]->held;
        }
        if (launch_moe_hetero_gemv1(a, devs, held, (int)w->pools.size(), pairs, w->info.device, stream)) return;
    }
    if (x_mode == 2 || tail) fail(MFQB_ERR_UNSUPPORTED, "mul_mat_id: this record's cohorts have no all-cohort single-row kernel");
    if (plan && gemm) {   // large batches: tensor-core tile kernel, `planes` holds the gathered f16 rows
        launch_x_gather_f16(x, x_mode == 1, plan->pair_order, x_per_pair ? 1 : routes, pairs, w->info.k, planes, stream);
        const int tiles = pairs / tile_m + std::min(pairs, w->info.n_experts);
        if (tiles > 65535) fail(MFQB_ERR_ARG, "mfqb_mul_mat_id: too many route tiles (%d)", tiles);
        for (size_t pi = 0; pi < w->pools.size(); ++pi) {
            const MoePool& pool = *w->pools[pi];
            if (!pool.held) continue;
            launch_nint_gemm_grouped(pool.d, planes, pairs, tile_m, plan->expert_bounds, plan->tile_bounds, plan->pair_order,
                                     static_cast<const int*>(w->d_expert_pool.p), static_cast<const int*>(w->d_expert_local.p),
                                     w->info.n_experts, (int)pi, w->padded / 16, ope, tiles, out, out_dtype, w->info.device, stream);
        }
        return;
    }
    if (plan && (tile_m == 8 || tile_m == 16) && moe_f16_tiles_ok(w)) {   // f16 tile kernel, all cohorts in one launch
        const int max_tiles_h = pairs / tile_m + std::min(pairs, w->info.n_experts);
        if (max_tiles_h > 65535) fail(MFQB_ERR_ARG, "mfqb_mul_mat_id: too many route tiles (%d)", max_tiles_h);
        GemvArgsB a{};
        a.y = out;
        a.ldy = ope;
        a.y_dtype = out_dtype;
        a.expert_pool = static_cast<const int*>(w->d_expert_pool.p);
        a.expert_local = static_cast<const int*>(w->d_expert_local.p);
        a.rb_per_expert = w->padded / 16;
        a.routes = routes;
        a.x_per_pair = x_per_pair ? 1 : 0;
        a.expert_bounds = plan->expert_bounds;
        a.tile_bounds = plan->tile_bounds;
        a.pair_order = plan->pair_order;
        a.n_experts = w->info.n_experts;
        NintDevB devs[16];
        int held[16];
        XFragArgs fa{};
        for (size_t pi = 0; pi < w->pools.size(); ++pi) {
            devs[pi] = w->pools[pi]->d;
            held[pi] = w->pools[pi]->held;
            fa.pool_t8[pi] = w->pools[pi]->d.t8;
            fa.pool_nchunks[pi] = w->pools[pi]->held ? w->pools[pi]->d.nchunks : 0;
        }
        fa.x = x;
        fa.x_f32 = x_mode == 1;
        fa.k = w->info.k;
        fa.nt = tile_m / 8;
        fa.tile_stride = moe_frag_tile_units(w, fa.nt);
        fa.expert_bounds = plan->expert_bounds;
        fa.tile_bounds = plan->tile_bounds;
        fa.pair_order = plan->pair_order;
        fa.expert_pool = static_cast<const int*>(w->d_expert_pool.p);
        fa.n_experts = w->info.n_experts;
        fa.routes = routes;
        fa.x_per_pair = x_per_pair ? 1 : 0;
        launch_x_frags(fa, in_rows, max_tiles_h, moe_max_nchunks(w), planes, &a.x16f, &a.x16_scale, stream);
        a.x16f_tile_stride = fa.tile_stride;
        if (launch_moe_hetero_tilesh(a, devs, held, (int)w->pools.size(), tile_m, max_tiles_h, w->info.device, stream)) return;
        fail(MFQB_ERR_UNSUPPORTED, "mul_mat_id: tiles of %d pairs do not fit the f16 tile kernel for this record", tile_m);
    }
    // quantised planes of the input rows, one set per distinct group size among the held cohorts
    const uint2* pool_xq[16] = {nullptr};
    const float2* pool_gtab[16] = {nullptr};
    if (plan) {
        for (size_t pi = 0; pi < w->pools.size(); ++pi) {
            const MoePool& pool = *w->pools[pi];
            if (!pool.held) continue;
            const PlaneSet* ps = nullptr;
            for (const PlaneSet& c : sets)
                if (c.gs == pool.d.gs) ps = &c;
            if (!ps) {
                PlaneSet n{pool.d.gs, nullptr, nullptr};
                launch_x_planes(pool.d, x, in_rows, planes_next, &n.xq, &n.gtab, stream, x_mode == 1);
                planes_next += (nint_bl_planes_bytes(pool.d, in_rows) + 255) / 256 * 256;
                sets.push_back(n);
                ps = &sets.back();
            }
            pool_xq[pi] = ps->xq;
            pool_gtab[pi] = ps->gtab;
        }
    }
    const int max_tiles = plan ? pairs / tile_m + std::min(pairs, w->info.n_experts) : 0;
    if (plan && max_tiles > 65535) fail(MFQB_ERR_ARG, "mfqb_mul_mat_id: too many route tiles (%d)", max_tiles);
    if (plan && w->pools.size() <= 16) {   // all cohorts in one launch when their codecs allow
        GemvArgsB a{};
        a.x = static_cast<const __nv_bfloat16*>(x);
        a.y = out;
        a.ldy = ope;
        a.y_dtype = out_dtype;
        a.expert_pool = static_cast<const int*>(w->d_expert_pool.p);
        a.expert_local = static_cast<const int*>(w->d_expert_local.p);
        a.rb_per_expert = w->padded / 16;
        a.routes = routes;
        a.x_per_pair = x_per_pair ? 1 : 0;
        a.expert_bounds = plan->expert_bounds;
        a.tile_bounds = plan->tile_bounds;
        a.pair_order = plan->pair_order;
        a.n_experts = w->info.n_experts;
        NintDevB devs[16];
        int held[16];
        for (size_t pi = 0; pi < w->pools.size(); ++pi) {
            devs[pi] = w->pools[pi]->d;
            held[pi] = w->pools[pi]->held;
        }
        if (launch_moe_hetero_tiles(a, devs, held, pool_xq, pool_gtab, (int)w->pools.size(), tile_m, max_tiles, w->info.device, stream)) return;
    }
    if (!plan && x_mode != 0) fail(MFQB_ERR_UNSUPPORTED, "mul_mat_id: the per-cohort single-row launches take bf16 activations");
    for (size_t pi = 0; pi < w->pools.size(); ++pi) {
        const MoePool& pool = *w->pools[pi];
        if (!pool.held) continue;
        GemvArgsB a{};
        a.w = pool.d;
        a.x = static_cast<const __nv_bfloat16*>(x);
        a.y = out;
        a.ldy = ope;
        a.y_dtype = out_dtype;
        a.expert_pool = static_cast<const int*>(w->d_expert_pool.p);
        a.expert_local = static_cast<const int*>(w->d_expert_local.p);
        a.pool = (int)pi;
        a.rb_per_expert = w->padded / 16;
        a.routes = routes;
        a.x_per_pair = x_per_pair ? 1 : 0;
        if (plan) {
            a.expert_bounds = plan->expert_bounds;
            a.tile_bounds = plan->tile_bounds;
            a.pair_order = plan->pair_order;
            a.n_experts = w->info.n_experts;
            a.xq_g = pool_xq[pi];
            a.gtab_g = pool_gtab[pi];
            launch_nint_bl_gemv_tiles(a, tile_m, max_tiles, w->info.device, stream);
            continue;
        }
        a.route_ids = ids;
        for (int p0 = 0; p0 < pairs; p0 += 32768) {   // gridDim.y limit
            GemvArgsB b = a;
            const int np = std::min(32768, pairs - p0);
            b.route_ids = ids + p0;
            b.y = static_cast<char*>(out) + (size_t)p0 * ope * (out_dtype == MFQB_F32 ? 4 : 2);
            if (p0 % routes) fail(MFQB_ERR_ARG, "mfqb_mul_mat_id: routes must divide 32768 for more than 32768 pairs");
            b.x = a.x + (size_t)(x_per_pair ? p0 : p0 / routes) * w->info.k;
            launch_nint_bl_gemv_routed(b, np, w->info.device, stream);
        }
    }
}

int mfqb_mul_mat_id(const mfqb_moe_weight* w, const void* x, int x_per_pair, const int32_t* ids, int tokens, int routes, void* out,
                    int out_dtype, mfqb_stream_t stream) {
    return guarded([&] {
        if (!w || !x || !ids || !out) fail(MFQB_ERR_ARG, "mfqb_mul_mat_id: null argument");
        if (tokens < 0 || routes < 1) fail(MFQB_ERR_ARG, "mfqb_mul_mat_id: bad sizes");
        if (out_dtype != MFQB_F32 && out_dtype != MFQB_BF16) fail(MFQB_ERR_ARG, "mfqb_mul_mat_id: bad output dtype");
        if (tokens == 0) return;
        DeviceGuard guard(w->info.device);
        const int pairs = tokens * routes;
        const int gemm_bn = moe_gemm_bn(w, pairs);
        const int tile_m = gemm_bn ? gemm_bn : moe_tile_m(w, pairs);
        if (tile_m) {   // larger batches: route plan in library scratch, batched or tile kernel over its tiles
            const size_t b_plan = PlanBufs::bytes(w->info.n_experts, pairs);
            const size_t b_in = gemm_bn ? nint_gemm_grouped_x_bytes(pairs, w->info.k) : moe_planes_bytes(w, x_per_pair ? pairs : tokens, pairs, tile_m);
            char* s = static_cast<char*>(scratch_get(w->info.device, b_plan + b_in, stream, 1));
            PlanBufs plan = PlanBufs::carve(s, w->info.n_experts);
            launch_route_plan(ids, pairs, w->info.n_experts, tile_m, plan.expert_bounds, plan.tile_bounds, plan.pair_order, stream);
            mul_mat_id_impl(w, x, x_per_pair, ids, tokens, routes, out, out_dtype, &plan, tile_m, s + b_plan, stream, gemm_bn != 0);
        } else {
            mul_mat_id_impl(w, x, x_per_pair, ids, tokens, routes, out, out_dtype, nullptr, 0, nullptr, stream);
        }
    });
}

// True when the all-cohort single-row kernel can run both matmuls of the FFN with nothing stored in
// between: SwiGLU formed while the down matmul loads, the weighted route sum in its epilogue.
static bool ffn_fused_tail_ok(const mfqb_moe_weight* down, int tokens, int pairs) {
    NintDevB devs[16];
    int held[16];
    if (down->pools.size() > 16 || pairs > 32768) return false;
    for (size_t pi = 0; pi < down->pools.size(); ++pi) {
        devs[pi] = down->pools[pi]->d;
        held[pi] = down->pools[pi]->held;
    }
    if (!moe_hetero_supported(devs, held, (int)down->pools.size())) return false;
    return (size_t)tokens * moe_hetero_gemv1_splits(down->padded / 16, pairs, down->info.device) * 4 <= kFfnCounterBytes;
}

// The FFN proper, on caller-provided scratch `s` laid out as
//   [route-sum counters (zero between calls) | gate|up products | activation | down products | route plan | planes].
static void moe_ffn_run(const mfqb_moe_weight* gate_up, const mfqb_moe_weight* down, const void* x, const int32_t* ids, const float* weights,
                        int tokens, int routes, void* y, int y_dtype, char* s, const FfnLayout& L, cudaStream_t stream) {
    const int f = gate_up->info.out_per_expert / 2, h = gate_up->info.k;
    const size_t pairs = (size_t)tokens * routes;
    float* gu = reinterpret_cast<float*>(s + L.o_gu);
    float* hid = reinterpret_cast<float*>(s + L.o_hid);
    float* dn = reinterpret_cast<float*>(s + L.o_dn);
    PlanBufs plan{};
    if (L.tiles) {   // one route plan serves both matmuls
        plan = PlanBufs::carve(s + L.o_plan, gate_up->info.n_experts);
        launch_route_plan(ids, (int)pairs, gate_up->info.n_experts, L.tile_m, plan.expert_bounds, plan.tile_bounds, plan.pair_order, stream);
    }
    char* planes = s + L.o_planes;
    mul_mat_id_impl(gate_up, x, 0, ids, tokens, routes, gu, MFQB_F32, L.tiles ? &plan : nullptr, L.tile_m, planes, stream, L.gemm);
    if (L.fused_tail) {   // decode sizes: the down matmul reads the gate|up products and ends in the route sum
        const FfnTail tail{weights, dn, reinterpret_cast<unsigned*>(s), y, y_dtype};
        mul_mat_id_impl(down, gu, 1, ids, tokens, routes, dn, MFQB_F32, nullptr, 0, nullptr, stream, false, 2, &tail);
        return;
    }
    if (!L.tiles) {   // cohorts without an all-cohort kernel: bf16 activation through the per-cohort launches
        launch_swiglu(gu, MFQB_F32, (int)pairs, f, hid, stream);
        mul_mat_id_impl(down, hid, 1, ids, tokens, routes, dn, MFQB_F32, nullptr, 0, nullptr, stream);
    } else {          // the activation stays float32: no rounding between the two matmuls
        launch_swiglu_f32(gu, (int)pairs, f, hid, stream);
        mul_mat_id_impl(down, hid, 1, ids, tokens, routes, dn, MFQB_F32, &plan, L.tile_m, planes + L.b_pgu, stream, L.gemm, 1);
    }
    launch_weighted_reduce(dn, MFQB_F32, weights, tokens, routes, h, y, y_dtype, stream);
}

static void check_ffn_args(const char* who, const mfqb_moe_weight* gate_up, const mfqb_moe_weight* down, int tokens, int routes) {
    const int h = gate_up->info.k, f2 = gate_up->info.out_per_expert, f = f2 / 2;
    if (f2 % 2 || down->info.k != f || down->info.out_per_expert != h || down->info.n_experts != gate_up->info.n_experts)
        fail(MFQB_ERR_ARG, "%s: gate_up [E, 2F, H] and down [E, H, F] shapes do not match", who);
    if (gate_up->info.device != down->info.device) fail(MFQB_ERR_ARG, "%s: weights live on different devices", who);
    if (routes < 1 || routes > 64) fail(MFQB_ERR_ARG, "%s: routes per token must be in [1, 64], got %d", who, routes);
    if ((long long)tokens * routes > INT_MAX) fail(MFQB_ERR_ARG, "%s: %d tokens x %d routes is more than the kernels index", who, tokens, routes);
}

static FfnLayout ffn_layout(const mfqb_moe_weight* gate_up, const mfqb_moe_weight* down, int tokens, int routes, bool allow_gemm) {
    FfnLayout L{};
    const int h = gate_up->info.k, f2 = gate_up->info.out_per_expert, f = f2 / 2;
    const size_t pairs = (size_t)tokens * routes;
    auto up256 = [](size_t v) { return (v + 255) / 256 * 256; };
    // large batches: both matmuls on the tensor-core tile kernel, when every cohort of both has one
    const int gemm_bn = allow_gemm ? std::min(moe_gemm_bn(gate_up, (int)pairs), moe_gemm_bn(down, (int)pairs)) : 0;
    L.gemm = gemm_bn != 0;
    L.tile_m = L.gemm ? gemm_bn : std::min(moe_tile_m(gate_up, (int)pairs), moe_tile_m(down, (int)pairs));
    L.tiles = L.tile_m != 0;
    L.fused_tail = !L.tiles && ffn_fused_tail_ok(down, tokens, (int)pairs) && ffn_fused_tail_ok(gate_up, tokens, (int)pairs);
    const size_t b_plan = L.tiles ? PlanBufs::bytes(gate_up->info.n_experts, pairs) : 0;
    L.b_pgu = L.gemm ? up256(nint_gemm_grouped_x_bytes((int)pairs, h)) : (L.tiles ? moe_planes_bytes(gate_up, tokens, (int)pairs, L.tile_m) : 0);
    const size_t b_pdn = L.gemm ? nint_gemm_grouped_x_bytes((int)pairs, f) : (L.tiles ? moe_planes_bytes(down, (int)pairs, (int)pairs, L.tile_m) : 0);
    L.o_gu = kFfnCounterBytes;
    L.o_hid = L.o_gu + up256(pairs * f2 * 4);
    L.o_dn = L.o_hid + up256(pairs * f * 4);
    L.o_plan = L.o_dn + up256(pairs * h * 4);
    L.o_planes = L.o_plan + b_plan;
    L.total = L.o_planes + L.b_pgu + b_pdn;
    return L;
}

int mfqb_moe_ffn(const mfqb_moe_weight* gate_up, const mfqb_moe_weight* down, const void* x, const int32_t* ids, const float* weights,
                 int tokens, int routes, void* y, int y_dtype, mfqb_stream_t stream) {
    return guarded([&] {
        if (!gate_up || !down || !x || !ids || !weights || !y) fail(MFQB_ERR_ARG, "mfqb_moe_ffn: null argument");
        check_ffn_args("mfqb_moe_ffn", gate_up, down, tokens, routes);
        if (tokens <= 0) return;
        DeviceGuard guard(gate_up->info.device);
        const FfnLayout L = ffn_layout(gate_up, down, tokens, routes, true);
        char* s = static_cast<char*>(scratch_get(gate_up->info.device, L.total, stream));
        moe_ffn_run(gate_up, down, x, ids, weights, tokens, routes, y, y_dtype, s, L, stream);
    });
}

#pragma GCC visibility pop
}  // extern "C"

// ---- expert FFN for callers that cannot allocate -------------------------------------------------
// Scratch for the intermediates lives in this fixed array inside the library image instead of a
// cudaMalloc'd buffer.  Every GPU that loads the library carries it until the process exits.
static __device__ __align__(256) unsigned char g_ffn_static_scratch[MFQB_STATIC_SCRATCH_BYTES];

namespace mfqb {
// The array's name is only a host-side stand-in; the device address is asked for once per device,
// with that device current, and cached.
static unsigned char* ffn_static_scratch(int device) {
    static std::mutex mu;
    static unsigned char* ptr[64] = {nullptr};
    std::lock_guard<std::mutex> lock(mu);
    if (device < 0 || device >= 64) fail(MFQB_ERR_ARG, "device index %d out of range", device);
    if (!ptr[device]) {
        void* p = nullptr;
        const cudaError_t e = cudaGetSymbolAddress(&p, g_ffn_static_scratch);
        if (e != cudaSuccess || !p) fail(MFQB_ERR_CUDA, "cudaGetSymbolAddress(static scratch): %s", cudaGetErrorString(e));
        ptr[device] = static_cast<unsigned char*>(p);
    }
    return ptr[device];
}
}  // namespace mfqb

extern "C" {
#pragma GCC visibility push(default)

int mfqb_moe_ffn_static(const mfqb_moe_weight* gate_up, const mfqb_moe_weight* down, const void* x, const int32_t* ids,
                        const float* weights, int tokens, int routes, void* y, int y_dtype, mfqb_stream_t stream) {
    return guarded([&] {
        if (!gate_up || !down || !x || !ids || !weights || !y) fail(MFQB_ERR_ARG, "mfqb_moe_ffn_static: null argument");
        check_ffn_args("mfqb_moe_ffn_static", gate_up, down, tokens, routes);
        if (tokens <= 0) return;
        // the tensor-core tile path keeps its own growing buffers: this entry point stays on the integer kernels
        const FfnLayout L = ffn_layout(gate_up, down, tokens, routes, false);
        if (L.total > (size_t)MFQB_STATIC_SCRATCH_BYTES)
            fail(MFQB_ERR_ARG,
                 "mfqb_moe_ffn_static: %d tokens x %d routes need %llu bytes of scratch, the built-in array holds %llu; "
                 "use mfqb_moe_ffn or fewer tokens per call",
                 tokens, routes, (unsigned long long)L.total, (unsigned long long)MFQB_STATIC_SCRATCH_BYTES);
        DeviceGuard guard(gate_up->info.device);
        unsigned char* s = ffn_static_scratch(gate_up->info.device);
        // The array still holds whatever the previous call left.  Only the route-sum counters must start at
        // zero (every other region is fully written before it is read); they are left zero by every
        // completed call, so this matters after a call that was interrupted.
        MFQB_CUDA(cudaMemsetAsync(s, 0, kFfnCounterBytes, stream));
        moe_ffn_run(gate_up, down, x, ids, weights, tokens, routes, y, y_dtype, reinterpret_cast<char*>(s), L, stream);
    });
}

#pragma GCC visibility pop
}  // extern "C"
