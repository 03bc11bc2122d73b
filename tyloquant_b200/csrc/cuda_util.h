// CUDA-side helpers shared by the .cu files of the library.
#pragma once
#include <cuda_runtime.h>

#include <mutex>

#include "common.h"

namespace mfqb {

#define MFQB_CUDA(expr)                                                                         \
    do {                                                                                        \
        const cudaError_t e_ = (expr);                                                          \
        if (e_ != cudaSuccess) ::mfqb::fail(MFQB_ERR_CUDA, "%s: %s", #expr, cudaGetErrorString(e_)); \
    } while (0)

// Makes `device` current for the scope and restores the previous device afterwards.
struct DeviceGuard {
    int prev = -1;
    explicit DeviceGuard(int device) {
        MFQB_CUDA(cudaGetDevice(&prev));
        if (prev != device) MFQB_CUDA(cudaSetDevice(device));
        else prev = -1;
    }
    ~DeviceGuard() {
        if (prev >= 0) cudaSetDevice(prev);
    }
};

int device_sm_count(int device);

// Owning device buffer.
struct DevBuf {
    void* p = nullptr;
    size_t bytes = 0;
    DevBuf() = default;
    DevBuf(const DevBuf&) = delete;
    DevBuf& operator=(const DevBuf&) = delete;
    DevBuf(DevBuf&& o) noexcept : p(o.p), bytes(o.bytes) {
        o.p = nullptr;
        o.bytes = 0;
    }
    void alloc(size_t n) {
        release();
        if (n) MFQB_CUDA(cudaMalloc(&p, n));
        bytes = n;
    }
    void upload(const void* src, size_t n) {
        alloc(n);
        if (n) MFQB_CUDA(cudaMemcpy(p, src, n, cudaMemcpyHostToDevice));
    }
    void release() {
        if (p) cudaFree(p);
        p = nullptr;
        bytes = 0;
    }
    ~DevBuf() { release(); }
};

// Library scratch that only ever grows: one block per device, handed to kernels that may still be
// in flight (or baked into a captured graph) when a later call needs more.  A larger request
// allocates a new block and keeps the old one alive until the process exits, so a pointer handed
// out once stays valid.  Growing allocates, which a stream capture does not allow: the call then
// fails with a message instead of breaking the capture.  Calls that share a block on one device
// must be ordered by their streams (the block holds one call's intermediates at a time).
struct GrowOnlyScratch {
    void* get(int device, size_t bytes, cudaStream_t stream, const char* what);

private:
    struct PerDevice {
        void* p = nullptr;
        size_t bytes = 0;
    };
    PerDevice dev_[64];
};

}  // namespace mfqb
