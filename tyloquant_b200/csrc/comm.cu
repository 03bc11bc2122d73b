// One-shot all-reduce of small float32 vectors over NVLink peer memory.
//
// The reference sums tensor-parallel / expert-parallel partial outputs with an in-place float32
// ncclAllReduce per row-parallel op, or by copying shards to the primary device and adding
// (cpp_runtime/mfq_decode.cpp:9009-9114).  At decode sizes (one to a few hundred rows of a few
// thousand floats) that is latency, not bandwidth: here every rank pushes its partial vector
// straight into a slot of every peer's buffer with plain stores, raises one flag per (peer, CTA),
// waits -- bounded -- for the same flags from its peers and adds the slots in rank order, so the
// result is bit-identical on every rank.  One kernel, no host round trip, NVSwitch carries
// world-1 copies of the vector per rank.
//
// Buffers are cudaMalloc'd per rank and shared between the one-process-per-GPU ranks through CUDA
// IPC handles (exchanged by the caller, e.g. over torch.distributed).  Two slot sets alternate
// with the call sequence number; a rank cannot run two calls ahead of a peer, because call s+1
// needs that peer's flag of call s+1, which the peer raises only after it finished call s.
// Every wait has a deadline; when it passes, the kernel records MFQB_ERR_TIMEOUT in a
// host-visible status word and returns, leaving the context usable.
#include <cuda_runtime.h>

#include <memory>
#include <vector>

#include "cuda_util.h"

namespace mfqb {

constexpr int kCommMaxWorld = 8;
constexpr int kCommMaxBlocks = 256;
constexpr int kCommBlockElems = 1024;   // floats per CTA

struct CommPeers {
    float* slots[kCommMaxWorld];        // per peer: [2 sets][world][max_elems]
    unsigned* flags[kCommMaxWorld];     // per peer: [2 sets][world][kCommMaxBlocks]
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

__global__ void __launch_bounds__(256) allreduce_oneshot_kernel(CommPeers peers, int rank, int world, unsigned long long max_elems,
                                                                const float* __restrict__ in, float* __restrict__ out,
                                                                unsigned long long n, unsigned seq, unsigned long long timeout_ns,
                                                                int* __restrict__ status) {
    const int set = seq & 1, b = blockIdx.x, tid = threadIdx.x;
    const unsigned long long lo = (unsigned long long)b * kCommBlockElems;
    const unsigned long long hi = lo + kCommBlockElems < n ? lo + kCommBlockElems : n;
    // push my part of the vector into slot `rank` of every rank (my own included)
    for (int p = 0; p < world; ++p) {
        float* dst = peers.slots[p] + ((size_t)set * world + rank) * max_elems;
        for (unsigned long long i = lo + tid; i < hi; i += blockDim.x) dst[i] = in[i];
    }
    __threadfence_system();
    __syncthreads();
    if (tid < world) st_release_sys(peers.flags[tid] + ((size_t)set * world + rank) * kCommMaxBlocks + b, seq);
    // wait for every rank's part of this block, with a deadline
    if (tid < world) {
        const unsigned* f = peers.flags[rank] + ((size_t)set * world + tid) * kCommMaxBlocks + b;
        const unsigned long long t0 = global_timer_ns();
        while (ld_acquire_sys(f) != seq) {
            if (global_timer_ns() - t0 > timeout_ns) {
                atomicExch(status, MFQB_ERR_TIMEOUT);
                break;
            }
        }
    }
    __syncthreads();
    const float* mine = peers.slots[rank] + (size_t)set * world * max_elems;
    for (unsigned long long i = lo + tid; i < hi; i += blockDim.x) {
        float acc = 0.f;
        for (int r = 0; r < world; ++r) acc += mine[(size_t)r * max_elems + i];
        out[i] = acc;
    }
}

}  // namespace mfqb

using namespace mfqb;

struct mfqb_comm {
    int rank = 0, world = 1, device = 0;
    uint64_t max_elems = 0;
    unsigned seq = 0;
    uint64_t timeout_ns = 2000000000ull;
    DevBuf local;                       // slots then flags of this rank
    void* peer_base[kCommMaxWorld] = {nullptr};
    bool opened[kCommMaxWorld] = {false};
    int* status_host = nullptr;         // pinned, mapped
    int* status_dev = nullptr;
    size_t slots_bytes() const { return (size_t)2 * world * max_elems * sizeof(float); }
    size_t flags_bytes() const { return (size_t)2 * world * kCommMaxBlocks * sizeof(unsigned); }
};

extern "C" {
#pragma GCC visibility push(default)

int mfqb_comm_create(int rank, int world, uint64_t max_elems, int device, mfqb_comm** out) {
    return guarded([&] {
        if (!out) fail(MFQB_ERR_ARG, "mfqb_comm_create: null output");
        if (world < 1 || world > kCommMaxWorld || rank < 0 || rank >= world)
            fail(MFQB_ERR_ARG, "mfqb_comm_create: rank %d / world %d out of range (world <= %d)", rank, world, kCommMaxWorld);
        if (max_elems == 0 || max_elems > (uint64_t)kCommMaxBlocks * kCommBlockElems)
            fail(MFQB_ERR_ARG, "mfqb_comm_create: max_elems must be in [1, %d]", kCommMaxBlocks * kCommBlockElems);
        auto c = std::make_unique<mfqb_comm>();
        c->rank = rank;
        c->world = world;
        c->device = device;
        c->max_elems = max_elems;
        DeviceGuard guard(device);
        c->local.alloc(c->slots_bytes() + c->flags_bytes());
        MFQB_CUDA(cudaMemset(c->local.p, 0, c->local.bytes));
        MFQB_CUDA(cudaHostAlloc((void**)&c->status_host, sizeof(int), cudaHostAllocMapped));
        *c->status_host = 0;
        MFQB_CUDA(cudaHostGetDevicePointer((void**)&c->status_dev, c->status_host, 0));
        c->peer_base[rank] = c->local.p;
        c->opened[rank] = false;
        *out = c.release();
    });
}

int mfqb_comm_handle(const mfqb_comm* c, void* handle64) {
    return guarded([&] {
        if (!c || !handle64) fail(MFQB_ERR_ARG, "mfqb_comm_handle: null argument");
        static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
        DeviceGuard guard(c->device);
        cudaIpcMemHandle_t h;
        MFQB_CUDA(cudaIpcGetMemHandle(&h, c->local.p));
        memcpy(handle64, &h, 64);
    });
}

int mfqb_comm_attach(mfqb_comm* c, int peer, const void* handle64) {
    return guarded([&] {
        if (!c || !handle64) fail(MFQB_ERR_ARG, "mfqb_comm_attach: null argument");
        if (peer < 0 || peer >= c->world || peer == c->rank) fail(MFQB_ERR_ARG, "mfqb_comm_attach: peer %d is not another rank of this communicator", peer);
        if (c->peer_base[peer]) fail(MFQB_ERR_ARG, "mfqb_comm_attach: peer %d is already attached", peer);
        DeviceGuard guard(c->device);
        cudaIpcMemHandle_t h;
        memcpy(&h, handle64, 64);
        void* p = nullptr;
        MFQB_CUDA(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
        c->peer_base[peer] = p;
        c->opened[peer] = true;
    });
}

int mfqb_comm_set_timeout_ms(mfqb_comm* c, int ms) {
    return guarded([&] {
        if (!c || ms < 1 || ms > 60000) fail(MFQB_ERR_ARG, "mfqb_comm_set_timeout_ms: 1..60000 ms");
        c->timeout_ns = (uint64_t)ms * 1000000ull;
    });
}

int mfqb_allreduce_f32(mfqb_comm* c, const float* in, float* out, uint64_t n, mfqb_stream_t stream) {
    return guarded([&] {
        if (!c || !in || !out) fail(MFQB_ERR_ARG, "mfqb_allreduce_f32: null argument");
        if (n == 0) return;
        if (n > c->max_elems) fail(MFQB_ERR_ARG, "mfqb_allreduce_f32: %llu elements exceed the communicator's %llu", (unsigned long long)n, (unsigned long long)c->max_elems);
        CommPeers peers{};
        for (int p = 0; p < c->world; ++p) {
            if (!c->peer_base[p]) fail(MFQB_ERR_ARG, "mfqb_allreduce_f32: rank %d has not been attached", p);
            peers.slots[p] = static_cast<float*>(c->peer_base[p]);
            peers.flags[p] = reinterpret_cast<unsigned*>(static_cast<char*>(c->peer_base[p]) + c->slots_bytes());
        }
        DeviceGuard guard(c->device);
        c->seq += 1;
        if (c->seq == 0) c->seq = 2;   // flags start at zero: never use 0 as a sequence number again
        const int grid = (int)((n + kCommBlockElems - 1) / kCommBlockElems);
        allreduce_oneshot_kernel<<<grid, 256, 0, stream>>>(peers, c->rank, c->world, c->max_elems, in, out, n, c->seq, c->timeout_ns,
                                                           c->status_dev);
        MFQB_CUDA(cudaGetLastError());
    });
}

int mfqb_comm_status(const mfqb_comm* c, int* status) {
    return guarded([&] {
        if (!c || !status) fail(MFQB_ERR_ARG, "mfqb_comm_status: null argument");
        *status = *static_cast<volatile int*>(c->status_host);
    });
}

int mfqb_comm_destroy(mfqb_comm* c) {
    return guarded([&] {
        if (!c) return;
        DeviceGuard guard(c->device);
        for (int p = 0; p < c->world; ++p)
            if (c->opened[p] && c->peer_base[p]) cudaIpcCloseMemHandle(c->peer_base[p]);
        if (c->status_host) cudaFreeHost(c->status_host);
        delete c;
    });
}

#pragma GCC visibility pop
}  // extern "C"
