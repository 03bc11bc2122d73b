// Device-side pieces of the one-shot NVLink reduction, shared by the stand-alone all-reduce
// kernel and the GEMV kernel that ends in a reduction.
#pragma once
#include <cstdint>

namespace mfqb {

constexpr int kCommMaxWorld = 8;
constexpr int kCommBlockElems = 1024;   // floats per CTA of the stand-alone kernel

// Where a thread pushes its values and where it waits for the peers': for every rank p the base of
// its slot array [2 sets][world][max_elems] of (value bits, sequence number) pairs.  A value and
// the number of the call it belongs to travel in one aligned 8-byte store, which is single-copy
// atomic, so no fence orders data against a flag: the receiver simply polls the pair until it
// carries the current call's number.  world == 0: no reduction.
struct PeerReduce {
    uint2* slots[kCommMaxWorld];
    int rank, world;
    // The call sequence number lives in device memory, so a launch carries no per-call argument and
    // can be replayed from a CUDA graph: a call uses *seq_dev + 1 and its last CTA stores it back.
    unsigned* seq_dev;
    unsigned* done_ctr;
    unsigned long long max_elems, timeout_ns;
    int* status;   // host-visible word: set to MFQB_ERR_TIMEOUT when a wait expires
};

// A (value, call number) pair travels as ONE 64-bit relaxed system-scope access: single-copy atomic by the
// memory model, so a reader never sees the value of one call with the number of another.
__device__ __forceinline__ void st_pair_sys(uint2* p, unsigned a, unsigned b) {
    const unsigned long long v = (unsigned long long)a | ((unsigned long long)b << 32);
    asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ uint2 ld_pair_sys(const uint2* p) {
    unsigned long long v;
    asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return make_uint2((unsigned)v, (unsigned)(v >> 32));
}
__device__ __forceinline__ unsigned long long global_timer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}

// This rank's value of element `elem` goes to slot `rank` of every rank (its own included).
__device__ __forceinline__ void peer_push(const PeerReduce& pr, unsigned seq, size_t elem, float v) {
    const size_t at = ((size_t)(seq & 1) * pr.world + pr.rank) * pr.max_elems + elem;
    for (int p = 0; p < pr.world; ++p) st_pair_sys(pr.slots[p] + at, __float_as_uint(v), seq);
}
// Sum over ranks of element `elem`, in rank order (the same bits on every rank).  Waits -- with a
// deadline -- for every rank's pair to carry this call's number; on expiry records the error and
// returns what it has.
__device__ __forceinline__ float peer_sum(const PeerReduce& pr, unsigned seq, size_t elem, int error_code) {
    const uint2* mine = pr.slots[pr.rank] + (size_t)(seq & 1) * pr.world * pr.max_elems + elem;
    float acc = 0.f;
    unsigned long long t0 = 0;
    for (int r = 0; r < pr.world; ++r) {
        const uint2* src = mine + (size_t)r * pr.max_elems;
        uint2 v = ld_pair_sys(src);
        unsigned spins = 0;
        while (v.y != seq) {
            if ((++spins & 31u) == 0) {
                const unsigned long long now = global_timer_ns();
                if (t0 == 0) t0 = now;
                if (now - t0 > pr.timeout_ns) {
                    atomicExch(pr.status, error_code);
                    break;
                }
            }
            v = ld_pair_sys(src);
        }
        if (v.y == seq) acc += __uint_as_float(v.x);
    }
    return acc;
}

// Sequence number of the call this kernel belongs to (never 0: flags start at zero).  Every CTA of
// the grid reads the same value: the store happens in peer_call_done, after all of them have read.
__device__ __forceinline__ unsigned peer_call_seq(const PeerReduce& pr) {
    __shared__ unsigned s_seq;
    if (threadIdx.x == 0) {
        // never 0 (slots start at zero), and the parity -- which selects the slot set -- must keep
        // alternating across the wrap: 0xFFFFFFFF (odd) is followed by 2 (even)
        const unsigned s = *reinterpret_cast<volatile unsigned*>(pr.seq_dev) + 1u;
        s_seq = s ? s : 2u;
    }
    __syncthreads();
    return s_seq;
}
// The last CTA of the grid to get here publishes the sequence number for the next call.
__device__ __forceinline__ void peer_call_done(const PeerReduce& pr, unsigned seq) {
    if (threadIdx.x == 0) {
        __threadfence();
        if (atomicAdd(pr.done_ctr, 1u) == gridDim.x * gridDim.y - 1u) {
            *reinterpret_cast<volatile unsigned*>(pr.done_ctr) = 0u;
            *reinterpret_cast<volatile unsigned*>(pr.seq_dev) = seq;
            __threadfence();
        }
    }
}

}  // namespace mfqb
