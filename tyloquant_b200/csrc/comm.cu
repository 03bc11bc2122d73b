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

#include "comm_dev.cuh"
#include "cuda_util.h"
#include "nint_blayout.h"

namespace mfqb {

__global__ void __launch_bounds__(256) allreduce_oneshot_kernel(const PeerReduce pr, const float* __restrict__ in, float* __restrict__ out,
                                                                unsigned long long n) {
    const int set = pr.seq & 1, b = blockIdx.x, tid = threadIdx.x, world = pr.world;
    const unsigned long long lo = (unsigned long long)b * kCommBlockElems;
    const unsigned long long hi = lo + kCommBlockElems < n ? lo + kCommBlockElems : n;
    // push my part of the vector into slot `rank` of every rank (my own included)
    for (int p = 0; p < world; ++p) {
        float* dst = pr.slots[p] + ((size_t)set * world + pr.rank) * pr.max_elems;
        for (unsigned long long i = lo + tid; i < hi; i += blockDim.x) dst[i] = in[i];
    }
    peer_signal_and_wait(pr, b, MFQB_ERR_TIMEOUT);
    const float* mine = pr.slots[pr.rank] + (size_t)set * world * pr.max_elems;
    for (unsigned long long i = lo + tid; i < hi; i += blockDim.x) {
        float acc = 0.f;
        for (int r = 0; r < world; ++r) acc += mine[(size_t)r * pr.max_elems + i];
        out[i] = acc;
    }
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

// Arguments of the next collective call of this communicator (advances its sequence number).
static PeerReduce next_call(mfqb_comm* c, const char* who) {
    PeerReduce pr{};
    for (int p = 0; p < c->world; ++p) {
        if (!c->peer_base[p]) fail(MFQB_ERR_ARG, "%s: rank %d has not been attached", who, p);
        pr.slots[p] = static_cast<float*>(c->peer_base[p]);
        pr.flags[p] = reinterpret_cast<unsigned*>(static_cast<char*>(c->peer_base[p]) + c->slots_bytes());
    }
    c->seq += 1;
    if (c->seq == 0) c->seq = 2;   // flags start at zero: never use 0 as a sequence number again
    pr.rank = c->rank;
    pr.world = c->world;
    pr.seq = c->seq;
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
        if (grid > kCommMaxBlocks) fail(MFQB_ERR_ARG, "mfqb_allreduce_f32: at most %d elements per call", kCommMaxBlocks * kCommBlockElems);
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
