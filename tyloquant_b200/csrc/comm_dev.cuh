// Device-side pieces of the one-shot NVLink reduction, shared by the stand-alone all-reduce
// kernel and the GEMV kernel that ends in a reduction.
#pragma once
#include <cstdint>

namespace mfqb {

constexpr int kCommMaxWorld = 8;
constexpr int kCommMaxBlocks = 512;     // CTAs of one call (one flag each per peer)
constexpr int kCommBlockElems = 1024;   // floats per CTA of the stand-alone kernel

// Where a CTA pushes its part of a vector and where it waits: for every rank p the base of its
// slot array [2 sets][world][max_elems] floats and of its flag array [2 sets][world][kCommMaxBlocks].
// world == 0: no reduction.
struct PeerReduce {
    float* slots[kCommMaxWorld];
    unsigned* flags[kCommMaxWorld];
    int rank, world;
    unsigned seq;
    unsigned long long max_elems, timeout_ns;
    int* status;   // host-visible word: set to MFQB_ERR_TIMEOUT when a wait expires
};

__device__ __forceinline__ void st_release_sys(unsigned* p, unsigned v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned* p) {
    unsigned v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ unsigned long long global_timer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}

// After a CTA has stored its values into slot `rank` of every peer (and fenced): thread t < world
// raises the CTA's flag at rank t and waits -- with a deadline -- for rank t's flag here.  All
// threads of the CTA must call it; on return the CTA may read the slots of its block.
__device__ __forceinline__ void peer_signal_and_wait(const PeerReduce& pr, int block, int error_code) {
    const int set = pr.seq & 1, tid = threadIdx.x;
    __threadfence_system();
    __syncthreads();
    if (tid < pr.world) {
        st_release_sys(pr.flags[tid] + ((size_t)set * pr.world + pr.rank) * kCommMaxBlocks + block, pr.seq);
        const unsigned* f = pr.flags[pr.rank] + ((size_t)set * pr.world + tid) * kCommMaxBlocks + block;
        const unsigned long long t0 = global_timer_ns();
        while (ld_acquire_sys(f) != pr.seq) {
            if (global_timer_ns() - t0 > pr.timeout_ns) {
                atomicExch(pr.status, error_code);
                break;
            }
        }
    }
    __syncthreads();
}

}  // namespace mfqb
