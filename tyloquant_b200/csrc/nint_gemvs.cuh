// Streamed single-row GEMV for NINT weights in the byte-lane layout: the decode hot path for a
// plain (unrouted) weight.
//
// Same arithmetic as the ring kernel of nint_gemv1_bl.cuh (activations quantised per group to
// 16-bit integers in two byte planes, int8 tensor-core mma with a block-diagonal B, scales in
// float32), organised for the memory system instead of for the matrix shape:
//
//   * Work is the flat sequence of (row-block, chunk) records in storage order.  The grid is one
//     CTA per SM; CTA b owns the contiguous range [I*b/G, I*(b+1)/G) of the I records, so all SMs
//     stream the same number of bytes whatever the matrix shape, and every warp takes a contiguous
//     part of that: one long run of consecutive addresses.
//   * A warp moves its records with one bulk asynchronous copy each (cp.async.bulk, completion
//     counted on an mbarrier) through a private ring; the first records are requested before the
//     kernel waits for its predecessor in the stream, since weights are constants.  A CTA takes
//     at most half an SM, so under programmatic dependent launch the next product's CTA is
//     resident and filling its ring while this one still streams.
//   * The activation row is quantised once per CTA into shared memory, laid out so that the B
//     fragments of the block-diagonal operand are plain loads: a lane reads either its group's
//     plane words or a block of zeros, no masks in the loop.
//   * A lane keeps float32 running sums for its two rows over a whole row-block segment; row
//     anchors, the reduction over the quad and the shared-memory hand-over happen once per
//     segment, not once per record.
//   * No CTA-wide barrier after staging.  A row-block's sixteen rows are finished by the last of
//     the warps that hold records of it (a shared-memory counter per row-block), which adds the
//     warps' segments in warp order and writes the output.  A row-block whose records straddle
//     CTAs is finished by the CTA that holds its first records, which reaches them last: the CTAs
//     that hold its later records reach theirs first and publish their partial rows to a small
//     global scratch, each value with a flag in one 8-byte store; the owner polls those pairs
//     (bounded), adds them in CTA order and clears them.  A publisher never waits for anybody.
#pragma once
#include "nint_gemv1_bl.cuh"
#include "tc05.cuh"

namespace mfqb {

struct GemvSArgs {
    NintDevB w;
    const void* x;          // [k] bf16 or f32
    int x_dtype;            // MFQB_BF16 / MFQB_F32
    void* y;                // [n]
    int y_dtype;
    uint2* fix_slots;       // [grid][16] (partial row bits, flag) of a row-block begun by an earlier CTA; all zero between calls
    int* error;             // device status word (host-visible): set when a bounded wait expires
    int stages;             // ring records per warp
    int maxseg;             // row-block segments one warp can touch
    int maxrb;              // row-blocks one CTA can touch
#ifdef MFQB_GEMVS_TRACE
    unsigned long long* trace;   // development builds only: [grid][16] timestamps of the kernel's phases
#endif
};

#ifdef MFQB_GEMVS_TRACE
#define MFQB_TRACE(slot) do { if (a.trace && threadIdx.x == 0) a.trace[blockIdx.x * 16 + (slot)] = global_timer_ns(); } while (0)
#else
#define MFQB_TRACE(slot) do { } while (0)
#endif

// Bytes of staged planes per group: T octets x 2 planes x one 16-byte row.
__host__ __device__ constexpr int gemvs_group_bytes(int t8) { return t8 * 32; }

__device__ __forceinline__ void bulk_copy_g2s(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smem_u32(smem_dst)), "l"(gsrc), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}

__device__ __forceinline__ uint4 lds128(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}

// One poll of an mbarrier phase (no "memory" clobber: the shared-memory reads that follow are
// volatile asm statements themselves, which the compiler keeps in order).
__device__ __forceinline__ bool mbar_try_once(uint32_t bar_addr, uint32_t parity) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(bar_addr), "r"(parity));
    return done != 0u;
}
// Slow path: keep polling, give up after `limit` polls.
static __device__ __noinline__ bool mbar_wait_slow(uint32_t bar_addr, uint32_t parity, uint32_t limit) {
#pragma unroll 1
    for (uint32_t it = 0; it < limit; ++it)
        if (mbar_try_once(bar_addr, parity)) return true;
    return false;
}
// Arms the barrier for `bytes` and starts the bulk copy that completes on it (issued by one lane).
// Weights are read once per call: the copy carries an evict-first L2 policy, so the stream does not
// push the activations, anchors and other small reused data out of L2.
__device__ __forceinline__ void ring_request(uint32_t slot_addr, const void* gsrc, uint32_t bytes, uint32_t bar_addr, uint64_t policy) {
    asm volatile(
        "mbarrier.arrive.expect_tx.shared::cta.b64 _, [%3], %2;\n\t"
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;"
        ::"r"(slot_addr), "l"(gsrc), "r"(bytes), "r"(bar_addr), "l"(policy));
}
__device__ __forceinline__ uint64_t l2_evict_first_policy() {
    uint64_t p;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
    return p;
}
__device__ __forceinline__ void prefetch_l2(const void* p) { asm volatile("prefetch.global.L2 [%0];" ::"l"(p)); }
// D (s32) = A (u8, 16x32) * B: first step of an accumulation (no input accumulator to clear first)
__device__ __forceinline__ void imma_u8u8_z(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.u8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
                 : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
}
__device__ __forceinline__ void imma_u8s8_z(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
                 : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
}

// Copies a kernel parameter into a register the compiler cannot re-derive from the parameter
// bank: a field first read late in the kernel would otherwise be fetched from the constant cache
// at that point, and after megabytes of weights have gone through L2 that fetch can miss all the
// way to HBM.  Every parameter is pinned at the top, while the kernel still waits for its
// predecessor anyway.
__device__ __forceinline__ uint32_t pin_u32(uint32_t v) {
    uint32_t r;
    asm volatile("mov.u32 %0, %1;" : "=r"(r) : "r"(v));
    return r;
}
__device__ __forceinline__ int pin_i32(int v) { return (int)pin_u32((uint32_t)v); }
template <class P>
__device__ __forceinline__ P* pin_ptr(P* p) {
    unsigned long long r;
    asm volatile("mov.u64 %0, %1;" : "=l"(r) : "l"((unsigned long long)(uintptr_t)p));
    return reinterpret_cast<P*>((uintptr_t)r);
}

__device__ __forceinline__ uint32_t lds32(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}
// Four 8x8 b16 matrices: lane l gives the address of row l%8 of matrix l/8; register m of lane
// 4q+c receives bytes 4c..4c+3 of row q of matrix m -- the B fragment layout of the int8 mma.
__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}

// Quantises the whole activation row into shared memory, as the 16-byte rows ldmatrix reads for
// the block-diagonal B operand.  In mma step (f, t) column n = 4f + o carries octet t of group
// 4f + o at k-bytes 8o .. 8o+7 of the 32, i.e. in the k-half o>>1 at byte offset 8*(o&1); the
// rest of the column is zero.  Row (g, t, plane) therefore holds the eight plane bytes of the
// octet at offset 8*(g&1) and zeros in its other half:
//   xq[((g*T + t)*2 + plane)*4 + 2*(g&1) + {0, 1}]   plane 0: low bytes, plane 1: high bytes
//   gtab[g] = (sx_g, sx_g * sum of the group's integers)
// One thread per octet (eight slots) of a group: pass 1 finds the groups' largest magnitudes
// (shared-memory atomic max on the float bits), pass 2 quantises with the group's power-of-two
// scale and adds up the integers, pass 3 writes the group table.  gmax / gsum: [ngp] words, zeroed
// by the caller (with a barrier) beforehand.
// Groups past the row's last group quantise zeros.  Every thread of the CTA must call it.
template <typename XT>
__device__ __forceinline__ void gemvs_load_octet(const XT* __restrict__ xrow, int k, int gs, int g, int t, bool fast, float (&v)[8]) {
    const int k0 = g * gs + 8 * t;
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = 0.f;
    if (8 * t >= gs || k0 >= k) return;
    if (fast && k0 + 8 <= k) {   // whole octet inside the group and the row, 16-byte aligned
        if constexpr (sizeof(XT) == 2) {
            const uint4 raw = __ldg(reinterpret_cast<const uint4*>(xrow + k0));
            v[0] = __uint_as_float(raw.x << 16); v[1] = __uint_as_float(raw.x & 0xFFFF0000u);
            v[2] = __uint_as_float(raw.y << 16); v[3] = __uint_as_float(raw.y & 0xFFFF0000u);
            v[4] = __uint_as_float(raw.z << 16); v[5] = __uint_as_float(raw.z & 0xFFFF0000u);
            v[6] = __uint_as_float(raw.w << 16); v[7] = __uint_as_float(raw.w & 0xFFFF0000u);
        } else {
            const float4 r0 = __ldg(reinterpret_cast<const float4*>(xrow + k0)), r1 = __ldg(reinterpret_cast<const float4*>(xrow + k0 + 4));
            v[0] = r0.x; v[1] = r0.y; v[2] = r0.z; v[3] = r0.w; v[4] = r1.x; v[5] = r1.y; v[6] = r1.z; v[7] = r1.w;
        }
        return;
    }
#pragma unroll
    for (int i = 0; i < 8; ++i)
        if (8 * t + i < gs && k0 + i < k) v[i] = (float)xrow[k0 + i];
}

// One octet of a bf16 row as four words of two bf16 each (zeros past the group or the row).
__device__ __forceinline__ uint4 gemvs_load_octet_raw(const __nv_bfloat16* __restrict__ xrow, int k, int gs, int g, int t, bool fast) {
    const int k0 = g * gs + 8 * t;
    if (8 * t >= gs || k0 >= k) return make_uint4(0u, 0u, 0u, 0u);
    if (fast && k0 + 8 <= k) return __ldg(reinterpret_cast<const uint4*>(xrow + k0));
    const unsigned short* xb = reinterpret_cast<const unsigned short*>(xrow);
    uint32_t e[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) e[i] = (8 * t + i < gs && k0 + i < k) ? (uint32_t)__ldg(xb + k0 + i) : 0u;
    return make_uint4(e[0] | (e[1] << 16), e[2] | (e[3] << 16), e[4] | (e[5] << 16), e[6] | (e[7] << 16));
}

// Quantises eight values with the group's scale exponent and stores the octet's two plane rows;
// returns the sum of the integers.
template <int T>
__device__ __forceinline__ int gemvs_quant_octet(const float (&v)[8], uint32_t eb, uint32_t sh, int g, int t, uint32_t* xq) {
    const float inv = __uint_as_float((268u - sh - min(eb, 254u)) << 23);
    constexpr float kMagic = 12582912.f;   // 1.5 * 2^23: the low 16 mantissa bits hold round(x * inv) in two's complement
    uint32_t f[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) f[i] = __float_as_uint(fmaf(v[i], inv, kMagic));
    int xs = 0;
    uint32_t lo[2], hi[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const uint32_t t01 = __byte_perm(f[4 * h], f[4 * h + 1], 0x5140), t23 = __byte_perm(f[4 * h + 2], f[4 * h + 3], 0x5140);
        lo[h] = __byte_perm(t01, t23, 0x5410);
        hi[h] = __byte_perm(t01, t23, 0x7632);
        xs = (int)__dp4a(lo[h], 0x01010101u, (unsigned)xs);          // unsigned low bytes
        xs += 256 * __dp4a((int)hi[h], 0x01010101, 0);               // signed high bytes
    }
    uint4* row = reinterpret_cast<uint4*>(xq + (size_t)(g * T + t) * 8);
    row[0] = (g & 1) ? make_uint4(0u, 0u, lo[0], lo[1]) : make_uint4(lo[0], lo[1], 0u, 0u);
    row[1] = (g & 1) ? make_uint4(0u, 0u, hi[0], hi[1]) : make_uint4(hi[0], hi[1], 0u, 0u);
    return xs;
}

// Long rows and float32 rows: two reads of x (the second hits L1).  Kept out of line: rarely taken.
template <int T, typename XT>
static __device__ __noinline__ void gemvs_stage_x_two_reads(const XT* __restrict__ xrow, int k, int gs, int units, bool fast, uint32_t* xq,
                                                            uint32_t* gmax, int* gsum) {
    constexpr uint32_t SH = sizeof(XT) == 2 ? 0u : 1u;
    for (int u = threadIdx.x; u < units; u += blockDim.x) {
        const int g = u / T, t = u - g * T;
        float v[8];
        gemvs_load_octet<XT>(xrow, k, gs, g, t, fast, v);
        uint32_t ab = 0u;   // largest magnitude as float bits (orders like the value; NaN is largest)
#pragma unroll
        for (int i = 0; i < 8; ++i) ab = max(ab, __float_as_uint(v[i]) & 0x7FFFFFFFu);
        if (ab) atomicMax(gmax + g, ab);
    }
    __syncthreads();
    for (int u = threadIdx.x; u < units; u += blockDim.x) {
        const int g = u / T, t = u - g * T;
        float v[8];
        gemvs_load_octet<XT>(xrow, k, gs, g, t, fast, v);
        const int xs = gemvs_quant_octet<T>(v, max(gmax[g] >> 23, 15u + kXScaleShift), SH, g, t, xq);
        if (xs) atomicAdd(gsum + g, xs);
    }
}

template <int T, typename XT>
__device__ __forceinline__ void gemvs_stage_x(const XT* __restrict__ xrow, int k, int gs, int ngp, uint32_t* xq, float2* gtab, uint32_t* gmax,
                                              int* gsum, const GemvSArgs& a) {
    // a bf16 magnitude rounds to at most 32640 on the 16-bit grid; a float32 one could reach 32768, so it gets one bit of headroom
    constexpr uint32_t SH = sizeof(XT) == 2 ? 0u : 1u;
    constexpr int MAXU = 4;   // octets a thread keeps in registers between the passes
    const int units = ngp * T;
    const bool fast = (gs & 7) == 0 && (reinterpret_cast<uintptr_t>(xrow) & 15) == 0;
    MFQB_TRACE(7);
    bool in_regs = false;
    if constexpr (sizeof(XT) == 2) {
        if (units <= MAXU * (int)blockDim.x) {   // one global read: the raw octets wait in registers for their group's maximum
            in_regs = true;
            const __nv_bfloat16* xb = reinterpret_cast<const __nv_bfloat16*>(xrow);
            uint4 raw[MAXU];
#pragma unroll
            for (int i = 0; i < MAXU; ++i) {
                const int u = threadIdx.x + i * blockDim.x;
                raw[i] = make_uint4(0u, 0u, 0u, 0u);
                if (u < units) raw[i] = gemvs_load_octet_raw(xb, k, gs, u / T, u % T, fast);
            }
#pragma unroll
            for (int i = 0; i < MAXU; ++i) {
                const int u = threadIdx.x + i * blockDim.x;
                // largest bf16 magnitude of the octet from the bit patterns (they order like the values; NaN is largest)
                const uint32_t m2 = __vimax3_s16x2(__vimax3_s16x2(0u, raw[i].x & 0x7FFF7FFFu, raw[i].y & 0x7FFF7FFFu), raw[i].z & 0x7FFF7FFFu,
                                                   raw[i].w & 0x7FFF7FFFu);
                const uint32_t ab = max(m2 & 0xFFFFu, m2 >> 16) << 16;
                if (u < units && ab) atomicMax(gmax + u / T, ab);
            }
            MFQB_TRACE(8);
            __syncthreads();
            MFQB_TRACE(9);
#pragma unroll
            for (int i = 0; i < MAXU; ++i) {
                const int u = threadIdx.x + i * blockDim.x;
                if (u < units) {
                    const int g = u / T, t = u - g * T;
                    const float v[8] = {__uint_as_float(raw[i].x << 16), __uint_as_float(raw[i].x & 0xFFFF0000u),
                                        __uint_as_float(raw[i].y << 16), __uint_as_float(raw[i].y & 0xFFFF0000u),
                                        __uint_as_float(raw[i].z << 16), __uint_as_float(raw[i].z & 0xFFFF0000u),
                                        __uint_as_float(raw[i].w << 16), __uint_as_float(raw[i].w & 0xFFFF0000u)};
                    const int xs = gemvs_quant_octet<T>(v, max(gmax[g] >> 23, 15u + kXScaleShift), SH, g, t, xq);
                    if (xs) atomicAdd(gsum + g, xs);
                }
            }
        }
    }
    if (!in_regs) gemvs_stage_x_two_reads<T, XT>(xrow, k, gs, units, fast, xq, gmax, gsum);
    MFQB_TRACE(10);
    __syncthreads();
    for (int g = threadIdx.x; g < ngp; g += blockDim.x) {
        const uint32_t eb = max(gmax[g] >> 23, 15u + kXScaleShift);
        // eb = 255: an infinity or NaN in the group; its scale becomes NaN and so does every output
        const float sx = __uint_as_float(eb >= 255u ? 0x7FC00000u : (eb - 14u - kXScaleShift + SH) << 23);
        gtab[g] = make_float2(sx, sx * (float)gsum[g]);
    }
}

// Index of the CTA whose range [I*b/G, I*(b+1)/G) holds record `it`.
// (32-bit arithmetic: the launcher only takes weights with total * (g + 1) < 2^31.)
__device__ __forceinline__ int gemvs_cta_of(int it, int total, int g) { return (int)(((unsigned)(it + 1) * (unsigned)g - 1u) / (unsigned)total); }

constexpr unsigned kGemvsPollLimit = 1u << 18;   // polls of a publisher's pair before the owner gives up

template <class C>
__device__ __forceinline__ void gemvs_body(const GemvSArgs& a, unsigned char* smem) {
    constexpr int T = C::T, WC = C::WC, SW = C::SW, REC = (WC + SW) * 32;
    constexpr bool EARLY = WC <= 24;   // narrow records: all code words into registers at once, ring slot refilled before the math
    static_assert(SW == 2 && C::HAS_MIN && !C::A_SIGNED, "streamed kernel: NINT codecs");
    const NintDevB& w = a.w;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, W = blockDim.x >> 5;
    const int q = lane >> 2, c = lane & 3;
    const int S = pin_i32(a.stages), nch = pin_i32(w.nchunks), ngp = nch * kChunkGroupsB;
    const int p_maxseg = pin_i32(a.maxseg), p_n = pin_i32(w.n), p_k = pin_i32(w.k), p_gs = pin_i32(w.gs);
    const int p_xdt = pin_i32(a.x_dtype), p_ydt = pin_i32(a.y_dtype), p_nrb = pin_i32(w.nrb);
    const void* p_x = pin_ptr(a.x);
    void* p_y = pin_ptr(a.y);
    uint2* p_slots = pin_ptr(a.fix_slots);
    int* p_err = pin_ptr(a.error);
    const uint32_t* p_items = pin_ptr(w.items);
    const uint32_t* p_anchors = pin_ptr(w.anchors);

    // shared memory: barriers | partial rows | group table | group maxima and sums | zero block | planes | rings
    uint64_t* bars_all = reinterpret_cast<uint64_t*>(smem);
    float* parts = reinterpret_cast<float*>(smem + (((size_t)W * S * 8 + 15) & ~(size_t)15));
    float2* gtab = reinterpret_cast<float2*>(parts + (size_t)W * p_maxseg * 16);
    uint32_t* gmax = reinterpret_cast<uint32_t*>(gtab + ngp);
    int* gsum = reinterpret_cast<int*>(gmax + ngp);
    int* rb_cnt = gsum + ngp;   // [maxrb] warps that have handed over their segment of each row-block of the CTA
    uint32_t* zero_blk = reinterpret_cast<uint32_t*>(rb_cnt + ((a.maxrb + 3) & ~3));
    uint32_t* xq = zero_blk + 72;   // 288 bytes of zeros: T rows of 32 bytes and one row more
    uint32_t* ring_all = reinterpret_cast<uint32_t*>((reinterpret_cast<uintptr_t>(xq + (size_t)ngp * T * 8) + 127) & ~(uintptr_t)127);
    uint64_t* bars = bars_all + warp * S;
    uint32_t* ring = ring_all + (size_t)warp * S * REC;

    __shared__ int wstart[33];   // first record of every warp of the CTA, then the CTA's end
    __shared__ int wrb[32];      // row-block of that record
    const int total = p_nrb * nch;
    const int G = gridDim.x, b = blockIdx.x;
    const int lo_b = (int)((unsigned)total * (unsigned)b / (unsigned)G), hi_b = (int)((unsigned)total * (unsigned)(b + 1) / (unsigned)G);
    const int n_b = hi_b - lo_b;
    const int w_lo = lo_b + (int)((unsigned)n_b * (unsigned)warp / (unsigned)W), w_hi = lo_b + (int)((unsigned)n_b * (unsigned)(warp + 1) / (unsigned)W);
    const int n_w = w_hi - w_lo;
    const int rb_main = w_lo / nch;   // row-block the warp starts in
    const int rb_first = lo_b / nch;  // first row-block of the CTA
    int rb = rb_main, ch = w_lo - rb_main * nch;
    MFQB_TRACE(0);
    if (lane == 0) {
        wstart[warp] = w_lo;
        wrb[warp] = rb_main;
        if (warp == W - 1) wstart[W] = hi_b;
        for (int s = 0; s < S; ++s) mbar_init(&bars[s], 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncwarp();
    pdl_launch_dependents_b();
    const uint32_t* src0 = p_items + (size_t)w_lo * REC;   // the warp's records are consecutive in memory
    const uint64_t policy = l2_evict_first_policy();
    if (lane == 0) {
        const int pre = min(S, n_w);
        for (int s = 0; s < pre; ++s) ring_request(smem_u32(ring + (size_t)s * REC), src0 + (size_t)s * REC, REC * 4, smem_u32(&bars[s]), policy);
    }
    // The activation row may still be written by the previous kernel, so it is not read yet -- but
    // asking L2 to fetch its lines is harmless (L2 is the point of coherence) and spares the first
    // read after the wait a trip to HBM.
    {
        const size_t xbytes = (size_t)p_k * (p_xdt == MFQB_F32 ? 4 : 2);
        const size_t line = ((size_t)b * blockDim.x + tid) * 128;
        if (line < xbytes) prefetch_l2(static_cast<const char*>(p_x) + line);
    }
    if (tid < 72) zero_blk[tid] = 0u;
    for (int g = tid; g < ngp; g += blockDim.x) { gmax[g] = 0u; gsum[g] = 0; }   // staging accumulators: cleared while the predecessor still runs
    for (int r = tid; r < a.maxrb; r += blockDim.x) rb_cnt[r] = 0;
    uint32_t an_lo = 0u, an_hi = 0u;   // anchors (f16 scale | f16 min << 16) of the lane's two rows: weights, so before the wait
    if (n_w > 0) {
        an_lo = __ldg(p_anchors + (size_t)rb * 16 + q);
        an_hi = __ldg(p_anchors + (size_t)rb * 16 + q + 8);
    }
    __syncthreads();
    MFQB_TRACE(1);
    pdl_wait_b();   // the activations come from the previous kernel
    MFQB_TRACE(2);
    gemvs_stage_x<T, __nv_bfloat16>(static_cast<const __nv_bfloat16*>(p_x), p_k, p_gs, ngp, xq, gtab, gmax, gsum, a);
    __syncthreads();
    MFQB_TRACE(3);

    // B operand by ldmatrix: lane l supplies the address of row n = l%8 (column n = group n of the
    // chunk) of matrix m = l/8 (m&1: k-half, m>>1: byte plane).  The row is live in the steps of
    // family n>>2 when the group's k-half (n&3)>>1 is m&1; everywhere else the lane points at zeros.
    const int bn = lane & 7, bm = lane >> 3;
    const bool blive = ((bn & 3) >> 1) == (bm & 1);
    constexpr uint32_t CHUNK_BYTES = kChunkGroupsB * T * 32;
    uint32_t pbase[2], pstep[2];
#pragma unroll
    for (int f = 0; f < 2; ++f) {
        const bool on = blive && (bn >> 2) == f;
        pbase[f] = on ? smem_u32(xq) + (uint32_t)((bn * T) * 2 + (bm >> 1)) * 16u : smem_u32(zero_blk);
        pstep[f] = on ? CHUNK_BYTES : 0u;   // dead rows stay on the zero block
    }
    const uint32_t gt_addr0 = smem_u32(gtab) + (uint32_t)(2 * c) * 8u;
    const uint32_t ring_addr = smem_u32(ring) + (uint32_t)lane * 4u;

    int stage = 0;
    uint32_t parity = 0;
    float acc_s_lo = 0.f, acc_s_hi = 0.f, acc_m_lo = 0.f, acc_m_hi = 0.f;
    float* my_parts = parts + (size_t)warp * p_maxseg * 16;
    bool failed = false;

    // Hands the warp's sums of the current row-block over; the last warp of the row-block to do so
    // finishes it: adds the segments in warp order, then publishes (the row-block began in an earlier
    // CTA), or collects what later CTAs published and writes the output rows.
    auto flush = [&]() {
        const float2 f_lo = __half22float2(*reinterpret_cast<const __half2*>(&an_lo));   // (ns, nm)
        const float2 f_hi = __half22float2(*reinterpret_cast<const __half2*>(&an_hi));
        float v_lo = f_lo.x * acc_s_lo - f_lo.y * acc_m_lo, v_hi = f_hi.x * acc_s_hi - f_hi.y * acc_m_hi;
        v_lo += __shfl_xor_sync(0xffffffffu, v_lo, 1);
        v_hi += __shfl_xor_sync(0xffffffffu, v_hi, 1);
        v_lo += __shfl_xor_sync(0xffffffffu, v_lo, 2);
        v_hi += __shfl_xor_sync(0xffffffffu, v_hi, 2);
        const int seg = rb - rb_main;
        if (c == 0) {
            my_parts[seg * 16 + q] = v_lo;
            my_parts[seg * 16 + q + 8] = v_hi;
        }
        acc_s_lo = acc_s_hi = acc_m_lo = acc_m_hi = 0.f;
        __threadfence_block();
        __syncwarp();
        const int r0 = rb * nch, r1 = r0 + nch, rs = max(lo_b, r0), re = min(hi_b, r1);
        // warps with records of this row-block: lane l answers for warp l
        const bool over = lane < W && wstart[lane + 1] > wstart[lane] && wstart[lane] < re && wstart[lane + 1] > rs;
        unsigned who = __ballot_sync(0xffffffffu, over);
        int old = 0;
        if (lane == 0) old = atomicAdd(rb_cnt + (rb - rb_first), 1);
        old = __shfl_sync(0xffffffffu, old, 0);
        if (old != __popc(who) - 1) return;   // another warp will finish it
        __threadfence_block();
        float v = 0.f;
        while (who) {
            const int wv = __ffs(who) - 1;
            who &= who - 1;
            if (lane < 16) v += parts[((size_t)wv * p_maxseg + (rb - wrb[wv])) * 16 + lane];
        }
        if (lane >= 16) return;
        if (rs != r0) {   // the row-block began in an earlier CTA: publish this CTA's share to it
            st_pair_sys(p_slots + (size_t)b * 16 + lane, __float_as_uint(v), 1u);
            return;
        }
        if (re != r1) {   // it continues in later CTAs: add what they published, in CTA order
            const int b_last = gemvs_cta_of(r1 - 1, total, G);
            for (int bb = b + 1; bb <= b_last; ++bb) {
                uint2* slot = p_slots + (size_t)bb * 16 + lane;
                uint2 pv = ld_pair_sys(slot);
                for (unsigned spins = 0; pv.y == 0u && spins < kGemvsPollLimit; ++spins) pv = ld_pair_sys(slot);
                if (pv.y == 0u) {
                    if (p_err) *p_err = MFQB_ERR_TIMEOUT;   // the publisher never came: give up on this row-block
                } else {
                    v += __uint_as_float(pv.x);
                    st_pair_sys(slot, 0u, 0u);
                }
            }
        }
        v *= kXScaleUndo;
        const int row = rb * 16 + lane;
        if (row < p_n) {
            if (p_ydt == MFQB_F32) reinterpret_cast<float*>(p_y)[row] = v;
            else reinterpret_cast<__nv_bfloat16*>(p_y)[row] = __float2bfloat16_rn(v);
        }
    };

    // Ring cursors as shared-memory addresses, advanced by constants: slot of the record being read,
    // its barrier, and the global address of the next record to request.
    const uint32_t bar0 = smem_u32(bars), slot0 = smem_u32(ring);
    uint32_t bar_addr = bar0, slot_addr = slot0;
    const uint32_t* src_next = src0 + (size_t)min(S, n_w) * REC;   // next record to request
    int to_request = n_w - min(S, n_w);
    for (int i = 0; i < n_w; ++i) {
        if (!mbar_try_once(bar_addr, parity)) {
            if (!mbar_wait_slow(bar_addr, parity, 1u << 22)) failed = true;
            if (__any_sync(0xffffffffu, failed)) break;
        }
        const uint32_t rec = slot_addr + (uint32_t)lane * 4u;   // this lane's word of row 0 of the record
        uint32_t qw[WC];
        uint32_t sw[SW];
        if constexpr (EARLY) {
#pragma unroll
            for (int j = 0; j < WC; ++j) qw[j] = lds32(rec + j * 128);
        }
#pragma unroll
        for (int j = 0; j < SW; ++j) sw[j] = lds32(rec + (WC + j) * 128);
        auto refill = [&]() {
            __syncwarp();   // every lane has read the slot
            if (to_request > 0) {
                if (lane == 0) ring_request(slot_addr, src_next, REC * 4, bar_addr, policy);
                src_next += REC;
                --to_request;
            }
        };
        if constexpr (EARLY) refill();

        const uint4 gtu = lds128(gt_addr0 + (uint32_t)ch * (kChunkGroupsB * 8));   // (sx, sx*X) of groups 2c, 2c+1
        const float4 gt = make_float4(__uint_as_float(gtu.x), __uint_as_float(gtu.y), __uint_as_float(gtu.z), __uint_as_float(gtu.w));
        int dlo[4], dhi[4];
#pragma unroll
        for (int f = 0; f < 2; ++f) {
            const uint32_t baddr = pbase[f] + (uint32_t)ch * pstep[f];
#pragma unroll
            for (int t = 0; t < T; ++t) {
                const int r = (f * T + t) * 4;
                uint32_t a0, a1, a2, a3;
                if constexpr (EARLY) {
                    typename C::Ctx ctx;
                    a0 = C::areg(qw, r, ctx, sw);
                    a1 = C::areg(qw, r + 1, ctx, sw);
                    a2 = C::areg(qw, r + 2, ctx, sw);
                    a3 = C::areg(qw, r + 3, ctx, sw);
                } else {
                    // wide records: the units that hold registers r .. r+3 straight from the ring slot
                    using BU = typename C::BU;
                    constexpr int U = BU::U, NP = BU::NP;
                    uint32_t aa[4];
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int unit = (r + e) / NP;
                        uint32_t uw[U];
#pragma unroll
                        for (int u = 0; u < U; ++u) uw[u] = lds32(rec + (unit * U + u) * 128);
                        aa[e] = BU::at(uw, (r + e) % NP);
                    }
                    a0 = aa[0]; a1 = aa[1]; a2 = aa[2]; a3 = aa[3];
                }
                uint32_t bl0, bl1, bh0, bh1;
                ldsm_x4(baddr + t * 32, bl0, bl1, bh0, bh1);
                if (f == 0 && t == 0) {
                    imma_u8u8_z(dlo, a0, a1, a2, a3, bl0, bl1);
                    imma_u8s8_z(dhi, a0, a1, a2, a3, bh0, bh1);
                } else {
                    imma_u8u8(dlo, a0, a1, a2, a3, bl0, bl1);
                    imma_u8s8(dhi, a0, a1, a2, a3, bh0, bh1);
                }
            }
        }
        if constexpr (!EARLY) refill();
        // D = 256 * high + low: sums of q * xi for rows (q, q+8) x groups (2c, 2c+1)
        const float d0 = (float)(dhi[0] * 256 + dlo[0]) * gt.x, d1 = (float)(dhi[1] * 256 + dlo[1]) * gt.z;
        const float d2 = (float)(dhi[2] * 256 + dlo[2]) * gt.x, d3 = (float)(dhi[3] * 256 + dlo[3]) * gt.z;
        float ss[4], sm[4];
        {
            typename C::Ctx ctx;
            C::scales(sw, ctx, ss, sm);
        }
        acc_s_lo = fmaf(ss[1], d1, fmaf(ss[0], d0, acc_s_lo));
        acc_s_hi = fmaf(ss[3], d3, fmaf(ss[2], d2, acc_s_hi));
        acc_m_lo = fmaf(sm[1], gt.w, fmaf(sm[0], gt.y, acc_m_lo));
        acc_m_hi = fmaf(sm[3], gt.w, fmaf(sm[2], gt.y, acc_m_hi));

        bar_addr += 8u;
        slot_addr += REC * 4;
        if (++stage == S) { stage = 0; parity ^= 1u; bar_addr = bar0; slot_addr = slot0; }
        ++ch;
        if (ch == nch || i + 1 == n_w) {   // the row-block, or the warp's range, ends here: hand the rows over
            flush();
            if (ch == nch) {
                ch = 0;
                ++rb;
                if (i + 1 < n_w) {
                    an_lo = __ldg(p_anchors + (size_t)rb * 16 + q);
                    an_hi = __ldg(p_anchors + (size_t)rb * 16 + q + 8);
                }
            }
        }
    }
    if (failed) {
        // a copy never arrived: record it, give the other copies in flight a bounded chance to land, leave
        if (lane == 0 && p_err) *p_err = MFQB_ERR_TIMEOUT;
        for (int s = 0; s < S; ++s) (void)mbar_wait(&bars[s], parity ^ (s < stage ? 1u : 0u), 1u << 16);
    }
    MFQB_TRACE(4);
#ifdef MFQB_GEMVS_TRACE
    if (a.trace && lane == 0) atomicMax(a.trace + blockIdx.x * 16 + 6, global_timer_ns());   // last warp of the CTA to get here
#endif
}

// Largest block per record width, two CTAs per SM: 64, 85 or 128 registers per thread.
__host__ __device__ constexpr int gemvs_max_threads(int wc) { return wc <= 18 ? 512 : (wc <= 24 ? 384 : 256); }

template <class C>
__global__ void __launch_bounds__(gemvs_max_threads(C::WC), 2) gemvs_kernel(const __grid_constant__ GemvSArgs a) {
    extern __shared__ __align__(16) unsigned char smem[];
    gemvs_body<C>(a, smem);
}

}  // namespace mfqb
