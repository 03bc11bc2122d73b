// One-shot all-reduce of small float32 vectors over NVLink peer memory.
//
// The reference sums tensor-parallel / expert-parallel partial outputs with an in-place float32
// ncclAllReduce per row-parallel op, or by copying shards to the primary device and adding
// (cpp_runtime/mfq_decode.cpp:9009-9114).  At decode sizes (one to a few hundred rows of a few
// thousand floats) that is latency, not bandwidth: here every rank pushes its partial vector
// straight into a slot of every peer's buffer, each value together with the number of the call in
// one 8-byte store, polls -- bounded -- its own slots until every rank's pair carries that number
// and adds them in rank order, so the result is bit-identical on every rank.  One kernel, no
// fence, no flag, no host round trip; NVSwitch carries world-1 copies of the vector per rank.
//
// Buffers are cudaMalloc'd per rank and shared between the one-process-per-GPU ranks through CUDA
// IPC handles (exchanged by the caller, e.g. over torch.distributed).  Two slot sets alternate
// with the call number; a rank cannot run two calls ahead of a peer, because call s+1 needs that
// peer's values of call s+1, which the peer sends only after it finished call s.  The call number
// is kept in device memory (the last CTA of a call advances it), so launches carry no per-call
// argument and replay from CUDA graphs.  Every wait has a deadline; when it passes, the kernel
// records MFQB_ERR_TIMEOUT in a host-visible status word and returns, leaving the context usable.
#include <cuda_runtime.h>

#include <memory>
#include <vector>

#include "comm_dev.cuh"
#include "cuda_util.h"
#include "nint_blayout.h"

namespace mfqb {

__global__ void __launch_bounds__(256) allreduce_oneshot_kernel(const PeerReduce pr, const float* __restrict__ in, float* __restrict__ out,
                                                                unsigned long long n) {
    const unsigned seq = peer_call_seq(pr);
    const unsigned long long lo = (unsigned long long)blockIdx.x * kCommBlockElems;
    const unsigned long long hi = lo + kCommBlockElems < n ? lo + kCommBlockElems : n;
    for (unsigned long long i = lo + threadIdx.x; i < hi; i += blockDim.x) peer_push(pr, seq, i, in[i]);
    for (unsigned long long i = lo + threadIdx.x; i < hi; i += blockDim.x) out[i] = peer_sum(pr, seq, i, MFQB_ERR_TIMEOUT);
    peer_call_done(pr, seq);
}

}  // namespace mfqb

using namespace mfqb;

namespace mfqb {
const NintDevB& weight_device_layout(const mfqb_weight* w);
int weight_device_index(const mfqb_weight* w);
void launch_bl_gemv_reduce(const NintDevB& w, const void* x, void* y, int y_dtype, int device, const PeerReduce& pr, cudaStream_t s);
}

struct mfqb_comm {
    int rank = 0, world = 1, device = 0;
    uint64_t max_elems = 0;
    DevBuf counters;                    // [0] sequence number of the last finished call, [1] CTAs done in the current one
    uint64_t timeout_ns = 2000000000ull;
    DevBuf local;                       // the slots of this rank
    void* peer_base[kCommMaxWorld] = {nullptr};
    bool opened[kCommMaxWorld] = {false};
    int* status_host = nullptr;         // pinned, mapped
    int* status_dev = nullptr;
    size_t slots_bytes() const { return (size_t)2 * world * max_elems * sizeof(uint2); }
};

extern "C" {
#pragma GCC visibility push(default)

int mfqb_comm_create(int rank, int world, uint64_t max_elems, int device, mfqb_comm** out) {
    return guarded([&] {
        if (!out) fail(MFQB_ERR_ARG, "mfqb_comm_create: null output");
        if (world < 1 || world > kCommMaxWorld || rank < 0 || rank >= world)
            fail(MFQB_ERR_ARG, "mfqb_comm_create: rank %d / world %d out of range (world <= %d)", rank, world, kCommMaxWorld);
        if (max_elems == 0 || max_elems > (1u << 22)) fail(MFQB_ERR_ARG, "mfqb_comm_create: max_elems must be in [1, %d]", 1 << 22);
        auto c = std::make_unique<mfqb_comm>();
        c->rank = rank;
        c->world = world;
        c->device = device;
        c->max_elems = max_elems;
        DeviceGuard guard(device);
        c->local.alloc(c->slots_bytes());
        MFQB_CUDA(cudaMemset(c->local.p, 0, c->local.bytes));
        c->counters.alloc(2 * sizeof(unsigned));
        MFQB_CUDA(cudaMemset(c->counters.p, 0, c->counters.bytes));
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

// Arguments of a collective call of this communicator (the sequence number advances on the device).
static PeerReduce next_call(mfqb_comm* c, const char* who) {
    PeerReduce pr{};
    for (int p = 0; p < c->world; ++p) {
        if (!c->peer_base[p]) fail(MFQB_ERR_ARG, "%s: rank %d has not been attached", who, p);
        pr.slots[p] = static_cast<uint2*>(c->peer_base[p]);
    }
    pr.rank = c->rank;
    pr.world = c->world;
    pr.seq_dev = static_cast<unsigned*>(c->counters.p);
    pr.done_ctr = pr.seq_dev + 1;
    pr.max_elems = c->max_elems;
    pr.timeout_ns = c->timeout_ns;
    pr.status = c->status_dev;
    return pr;
}

int mfqb_allreduce_f32(mfqb_comm* c, const float* in, float* out, uint64_t n, mfqb_stream_t stream) {
    return guarded([&] {
        if (!c || !in || !out) fail(MFQB_ERR_ARG, "mfqb_allreduce_f32: null argument");
        if (n == 0) return;
        if (n > c->max_elems) fail(MFQB_ERR_ARG, "mfqb_allreduce_f32: %llu elements exceed the communicator's %llu", (unsigned long long)n, (unsigned long long)c->max_elems);
        DeviceGuard guard(c->device);
        const int grid = (int)((n + kCommBlockElems - 1) / kCommBlockElems);
        const PeerReduce pr = next_call(c, "mfqb_allreduce_f32");
        allreduce_oneshot_kernel<<<grid, 256, 0, stream>>>(pr, in, out, n);
        MFQB_CUDA(cudaGetLastError());
    });
}

// Row-parallel product that ends in the reduction: y = sum over ranks of (x_shard * W_shard^T).
// Every rank holds a K-slice of the weight (same rows) and the matching slice of x; the GEMV
// kernel's own epilogue pushes its float32 partial rows into every peer's slots, signals, waits
// for the peers' parts of the same rows and writes the summed row: one kernel per rank, no
// partial vector in HBM, no second launch.
int mfqb_mul_mat_allreduce(const mfqb_weight* w, const void* x, int m, mfqb_comm* c, void* y, int y_dtype, mfqb_stream_t stream) {
    return guarded([&] {
        if (!w || !x || !c || !y) fail(MFQB_ERR_ARG, "mfqb_mul_mat_allreduce: null argument");
        if (m < 1) fail(MFQB_ERR_ARG, "mfqb_mul_mat_allreduce: m must be >= 1");
        if (y_dtype != MFQB_F32 && y_dtype != MFQB_BF16) fail(MFQB_ERR_ARG, "mfqb_mul_mat_allreduce: bad output dtype");
        const NintDevB& d = weight_device_layout(w);
        if (weight_device_index(w) != c->device) fail(MFQB_ERR_ARG, "mfqb_mul_mat_allreduce: weight and communicator live on different devices");
        if ((uint64_t)d.n > c->max_elems) fail(MFQB_ERR_ARG, "mfqb_mul_mat_allreduce: %d rows exceed the communicator's %llu elements", d.n, (unsigned long long)c->max_elems);
        DeviceGuard guard(c->device);
        const size_t ysz = y_dtype == MFQB_F32 ? 4 : 2;
        for (int i = 0; i < m; ++i) {   // one activation row per call of the fused kernel
            const PeerReduce pr = next_call(c, "mfqb_mul_mat_allreduce");
            launch_bl_gemv_reduce(d, static_cast<const char*>(x) + (size_t)i * d.k * 2, static_cast<char*>(y) + (size_t)i * d.n * ysz, y_dtype,
                                  c->device, pr, stream);
        }
    });
}

// Recovery after MFQB_ERR_TIMEOUT: the ranks' device-side call numbers may differ (a rank that
// timed out advanced alone).  Every rank calls this with none of its collectives in flight; it
// clears this rank's slots, call number and status.  The ranks must then meet on the host (a
// barrier of the caller's process group) before the next collective, so that no rank pushes into
// slots a peer has yet to clear.
int mfqb_comm_reset(mfqb_comm* c) {
    return guarded([&] {
        if (!c) fail(MFQB_ERR_ARG, "mfqb_comm_reset: null argument");
        DeviceGuard guard(c->device);
        MFQB_CUDA(cudaDeviceSynchronize());
        MFQB_CUDA(cudaMemset(c->local.p, 0, c->local.bytes));
        MFQB_CUDA(cudaMemset(c->counters.p, 0, c->counters.bytes));
        *c->status_host = 0;
    });
}

// Development hook for tests: sets the device-side call number (e.g. just below the 32-bit wrap).
int mfqb_comm_debug_set_seq(mfqb_comm* c, unsigned seq) {
    return guarded([&] {
        if (!c) fail(MFQB_ERR_ARG, "mfqb_comm_debug_set_seq: null argument");
        DeviceGuard guard(c->device);
        MFQB_CUDA(cudaDeviceSynchronize());
        MFQB_CUDA(cudaMemcpy(c->counters.p, &seq, sizeof(unsigned), cudaMemcpyHostToDevice));
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
