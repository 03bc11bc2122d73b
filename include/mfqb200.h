/* mfqb200 -- C ABI of the B200-native MFQ packed-weight execution path.
 *
 * Every function returns an int status (MFQB_OK == 0).  On failure a thread-local
 * message is available from mfqb_last_error().  No exception crosses this boundary.
 * Device work is enqueued on the caller's stream (a cudaStream_t passed as
 * mfqb_stream_t; NULL = the legacy default stream) and is asynchronous unless a
 * function says otherwise.  Handles are opaque and owned by the library until the
 * matching *_free / *_close call.  There is no CPU execution path: a call that needs
 * a GPU fails with MFQB_ERR_CUDA when none is usable.
 *
 * The comments cite the interface of the reference runtime that each entry point
 * stands in for (paths inside the reference project).
 */
#ifndef MFQB200_H
#define MFQB200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct CUstream_st* mfqb_stream_t; /* == cudaStream_t */

enum {
    MFQB_OK = 0,
    MFQB_ERR_ARG = 1,         /* bad argument (null pointer, size out of range, wrong handle) */
    MFQB_ERR_FORMAT = 2,      /* malformed or truncated file / blob */
    MFQB_ERR_UNSUPPORTED = 3, /* well-formed, but a dtype / profile outside this path */
    MFQB_ERR_CUDA = 4,        /* CUDA runtime error (message holds the CUDA error string) */
    MFQB_ERR_IO = 5,          /* file system error */
    MFQB_ERR_TIMEOUT = 6      /* a bounded device-side wait ran out (multi-GPU paths) */
};

enum { MFQB_F32 = 0, MFQB_BF16 = 1 }; /* element types of activations / outputs */

enum { MFQB_FAMILY_NINT = 1, MFQB_FAMILY_NVQ = 2 };

const char* mfqb_last_error(void);
int mfqb_version(void);

/* ---------------------------------------------------------------------------------
 * MFQ container.  Replaces MfqFile (cpp_runtime/mfq_decode.cpp:1294-1527) and the
 * Python reader (mfq/formats/io.py:782-831): "MFQ1", version, arch, optional extra
 * metadata, record table {name, dtype, nbytes}, blobs back to back.  A file whose
 * length differs from the end of the last blob is rejected.  Shards named
 * "<stem>-%05d-of-%05d.mfq" are opened together when the first shard is given
 * (cpp_runtime/mfq_decode.cpp:1359-1427).
 * --------------------------------------------------------------------------------- */
typedef struct mfqb_file mfqb_file;

int mfqb_file_open(const char* path, mfqb_file** out);
int mfqb_file_open_memory(const void* image, uint64_t nbytes, mfqb_file** out); /* copies */
int mfqb_file_close(mfqb_file* f);
int mfqb_file_header(const mfqb_file* f, uint32_t* version, const char** arch, int* n_extra,
                     int* n_records);
int mfqb_file_extra(const mfqb_file* f, int i, const char** key, const char** json);
int mfqb_file_record(const mfqb_file* f, int i, const char** name, const char** dtype,
                     uint64_t* nbytes);
int mfqb_file_find(const mfqb_file* f, const char* name, int* index); /* -1 if absent */
/* Pointer to the record's blob inside the mapping (valid until mfqb_file_close). */
int mfqb_file_blob(const mfqb_file* f, int i, const void** data, uint64_t* nbytes);

/* ---------------------------------------------------------------------------------
 * Dense quantized weights.  Replaces unpack_nint / unpack_nvq + the to-device copies
 * (cpp_runtime/mfq_decode.cpp:1546-1589, 2268-2293, 3756-4013, 4121-4139) and the
 * packed-domain tensor-parallel slicers slice_nint_cpu_output / _input_groups /
 * slice_nvq_cpu (cpp_runtime/mfq_decode.cpp:1663-1744, 3579-3677).
 *
 * dtype is the record's label ("NINT2".."NINT8", "NVQ3", "NVQ3J-512", "NVQ3J",
 * "NIQ3").  The blob is decoded on the host, re-laid into the device format and
 * uploaded to `device`; the call returns after the upload has completed.
 *
 * axis: 0 = output rows [begin,end), 1 = input columns [begin,end).  Input slices must
 * start on a group boundary (NINT) / a multiple of 24 (NVQ); begin=0,end=-1 = whole.
 * --------------------------------------------------------------------------------- */
typedef struct mfqb_weight mfqb_weight;

typedef struct mfqb_weight_info {
    int family;          /* MFQB_FAMILY_* */
    int bits;            /* NINT code width / NVQ index width */
    int groupsize;
    int sub_bits;
    int64_t n;           /* output rows held by this handle */
    int64_t k;           /* input columns held by this handle */
    int device;
    int jsc_banks;       /* NVQ-JSC codebook banks, 0 otherwise */
    uint64_t payload_bytes; /* algorithmic bytes: the file streams of this (slice of the)
                               tensor, header excluded -- the roofline numerator */
    uint64_t device_bytes;  /* bytes this handle actually holds in HBM */
} mfqb_weight_info;

int mfqb_weight_from_blob(const char* dtype, const void* blob, uint64_t nbytes, int device,
                          mfqb_weight** out);
int mfqb_weight_from_blob_slice(const char* dtype, const void* blob, uint64_t nbytes, int axis,
                                int64_t begin, int64_t end, int device, mfqb_weight** out);
int mfqb_weight_info_get(const mfqb_weight* w, mfqb_weight_info* info);
/* A second handle with its own device copy of the same weight, on the same device (device-to-device
 * copy: the host-side re-layout is not repeated).  No counterpart in the reference. */
int mfqb_weight_clone(const mfqb_weight* w, mfqb_weight** out);
int mfqb_weight_free(mfqb_weight* w);

/* Reference decoder on the GPU: writes the [n, k] row-major dequantized tensor.
 * out_dtype MFQB_F32 is bit-identical to nint_quant.dequantize / nvq_quant.dequantize /
 * dequantize_nvq_jsc (mfq/quantize/nint_quant.py:896-908, nvq_quant.py:612-626,
 * nvq_jsc.py:1053-1079); MFQB_BF16 is the nearest-even rounding of that.
 * Stands in for dequant_full_packed_* / nvq_dequant_kernel
 * (mfq/kernels/cuda/nint_matmul.cu:136-161,442-481, nvq_matmul.cu:421-471). */
int mfqb_dequant(const mfqb_weight* w, void* out, int out_dtype, mfqb_stream_t stream);

/* y[m, n] = x[m, k] . W^T.  x is row-major bf16 with exactly k columns; y is row-major [m, n] in
 * y_dtype.  Any m >= 1 is accepted.  m <= 16 (and every m for lattice weights) runs the
 * weight-streaming kernels: the weights stay integer codes on the int8 tensor cores, x is quantised
 * inside the kernel, group by group, to 16-bit integers with a power-of-two scale (exact for a bf16
 * value unless it lies more than 2^7 below its group's largest magnitude; the product is within
 * 1e-5 relative L2 of the float32 reference), sums are exact in int32 and the scales are applied
 * in float32.  Larger m for NINT runs the tcgen05 tile kernel (f16 operands, float32 accumulation).
 * An infinity or NaN in x makes the outputs NaN (on the tile kernel, finite magnitudes beyond
 * 65504 saturate to +-65504 in the f16 copy of x).
 * Library scratch: m >= 2 uses a per-device buffer (quantised planes, or the f16 copy of x) that
 * only ever grows -- a block handed to a kernel or baked into a captured graph stays allocated.
 * Growing calls cudaMalloc, so the first call with a given (or larger) m on a device must come
 * outside stream capture; inside a capture it fails with MFQB_ERR_ARG instead.  The buffer holds
 * one call's data at a time: calls with m >= 2 on one device must be ordered by their streams.
 * A single-row (m = 1) product of a NINT weight uses a few KB of scratch owned by the weight
 * handle: two such products of the SAME weight must not overlap on the GPU.
 * Stands in for nint_matmul / nvq_matmul / QuantLinear::forward
 * (cpp_runtime/mfq_decode.cpp:8130-8315, 7884-7932, 9209). */
int mfqb_mul_mat(const mfqb_weight* w, const void* x_bf16, int m, void* y, int y_dtype,
                 mfqb_stream_t stream);

/* One activation row x [1, k] against up to 8 NINT weights of one shape class (same code width,
 * group size and k; the row counts may differ) in ONE launch: ys[i] [1, n_i] = x . W_i^T.  What a
 * decoder does for q|k|v and gate|up -- the reference's NintLinearGroup / nvq_matmul_multi2
 * (cpp_runtime/mfq_decode.cpp:8618-8743, 7981-8070).  Same arithmetic as mfqb_mul_mat with m = 1. */
int mfqb_mul_mat_multi(const mfqb_weight* const* ws, int count, const void* x_bf16, void* const* ys,
                       int y_dtype, mfqb_stream_t stream);

/* Down projection of a gated FFN with the activation fused: gate_up [m, 2k] float32 (gate columns
 * first), y [m, n] = (up * gate / (1 + exp(-gate))) . W^T  (the reference's mul_mat_swiglu /
 * fused_swiglu_matmul, mfq/kernels/cuda/glu.cuh:6-17 + the linear call that follows it).  For m = 1
 * on NINT weights the activation is computed inside the single-row kernel as it loads the row; other
 * cases run the activation kernel into library scratch, then mfqb_mul_mat. */
int mfqb_mul_mat_swiglu(const mfqb_weight* w, const void* gate_up_f32, int m, void* y, int y_dtype,
                        mfqb_stream_t stream);

/* Gate|up projection of a gated FFN with the activation in the epilogue.  The weight's rows come in
 * 16-row blocks that alternate gate rows and up rows (block 2i = gate rows 16i .. 16i+15, block
 * 2i+1 = the up rows of the same indices: a row permutation applied when the fused weight is
 * packed); y [m, n / 2] = up * gate / (1 + exp(-gate)).  The same composition as
 * mfqb_mul_mat_swiglu (mfq/kernels/cuda/glu.cuh:6-17) with the activation on the producing side,
 * so the following down projection is a plain mfqb_mul_mat.  m = 1 on NINT weights runs in the
 * single-row kernel; other cases take the product into library scratch and apply the activation. */
int mfqb_mul_mat_glu(const mfqb_weight* w, const void* x_bf16, int m, void* y, int y_dtype,
                     mfqb_stream_t stream);

/* Residual add, RMSNorm and a single-row product in one launch (what a decoder block does before q|k|v
 * and before gate|up; the reference runs rmsnorm and the linear as two kernels,
 * cpp_runtime/mfq_decode.cpp:12210-12400): h [k] float32 residual row, delta [k] float32 or null,
 * gamma [k] float32; y [1, n] = W . ((h + delta) / rms(h + delta) * gamma), or with gated != 0 the
 * gated form of mfqb_mul_mat_glu ([1, n / 2]).  When h_out is not null it receives h + delta (it must
 * be another buffer than h).  NINT weights, k a multiple of 4.  Every CTA of the product normalises the
 * row for itself, which pays for short outputs; for the projections of an 8B-shaped decoder block the
 * separate normalisation kernel measured faster, and the decoder below keeps it. */
int mfqb_mul_mat_rmsnorm(const mfqb_weight* w, const float* h, const float* delta, const float* gamma, float eps,
                         float* h_out, void* y, int y_dtype, int gated, mfqb_stream_t stream);

/* Tuning switches, for measurements.  "gemv1_kernel": which kernel a single-row product of a plain
 * NINT weight takes -- 0 by shape (default), 1 the per-warp ring kernel, 2 the streamed kernel.
 * "moe_f16_tiles_from_x2": twice the average number of (token, route) pairs per expert from which
 * the expert matmuls take the f16 tile kernel instead of the integer tiles (default 4).
 * "gemm_plan": 0 = ring sizes of the tensor-core tile kernel by shape (default), 1 = 32-column
 * activation stages with a two-chunk weight ring for every shape.
 * No counterpart in the reference (its switches are MFQ_* environment variables,
 * docs/developer-architecture-and-operator-reference.md:1048-1078). */
int mfqb_tune(const char* key, int value);

/* Status word of the device-side bounded waits of the tile kernel on `device`: 0, or
 * MFQB_ERR_TIMEOUT when a wait inside a kernel ran out (the kernel then returned early and
 * its output is not valid).  Reads a host-mapped word; does not synchronise. */
int mfqb_device_status(int device, int* status);

/* Same product with host buffers: copies x to the device, runs, copies y back and
 * waits.  (The reference runtime keeps activations on the device; this entry point is
 * what a host-side caller such as the numpy runtime mfq/runtime/linear.py:37-42 uses.) */
int mfqb_mul_mat_host(const mfqb_weight* w, const void* x_bf16_host, int m, void* y_host,
                      int y_dtype);
/* The same for `count` weights of one device in one call, weight i with its own xs_host[i]
 * [m, k_i] and ys_host[i] [m, n_i]: everything is enqueued back to back and the call waits once
 * (the host-side form of a group of linears that run together, QuantLinearGroup / NintLinearGroup,
 * cpp_runtime/mfq_decode.cpp:8618-8743).  Pinned, mapped buffers are read and written in place. */
int mfqb_mul_mat_host_multi(const mfqb_weight* const* ws, int count, const void* const* xs_bf16_host,
                            int m, void* const* ys_host, int y_dtype);

/* ---------------------------------------------------------------------------------
 * Tensor-parallel slice planner.  Same results and the same rejections as
 * plan_tensor_parallel_slices / validate_tensor_parallel_slices
 * (cpp_runtime/tensor_parallel.h:23-118) and tensor_parallel_granularity
 * (cpp_runtime/mfq_decode.cpp:9445-9461).  weights may be NULL (equal split).
 * begins/ends receive n_devices entries each.
 * --------------------------------------------------------------------------------- */
int mfqb_tp_plan(int64_t extent, int64_t granularity, int n_devices, const double* weights,
                 int64_t* begins, int64_t* ends);
int mfqb_tp_validate(int64_t extent, int64_t granularity, int n_slices, const int64_t* begins,
                     const int64_t* ends);
int mfqb_tp_granularity(int64_t extent, int64_t preferred, int n_devices, int64_t* out);

/* ---------------------------------------------------------------------------------
 * Mixture-of-experts routing.
 *
 * mfqb_moe_topk replaces moe_topk_cuda (mfq/kernels/cuda/moe.cu:124-263, 3552-3637):
 * per token, the k experts with the highest score, in descending score order, ties to the
 * smaller expert id, NaN logits ranking last.  mode: 0 softmax over all experts, 1 sigmoid,
 * 2 sqrt(softplus), 3 "delayed softmax" (select on raw logits, softmax over the selected k --
 * the default of the reference FFN, cpp_runtime/mfq_decode.cpp:10483).  bias (may be NULL)
 * is added to the score used for selection only.  With modes 0-2 `normalize` divides the k
 * weights by max(sum, norm_floor).  Weights are finally multiplied by `scale`.
 * logits: device float32 [tokens, experts]; ids: device int32 [tokens, k]; weights: device
 * float32 [tokens, k].  k <= 16, experts <= 4096.
 *
 * mfqb_moe_route_plan replaces build_moe_route_plan / moe_build_expert_map_cuda
 * (cpp_runtime/mfq_decode.cpp:2681-2708, mfq/kernels/cuda/moe.cu:472-542, 3676-3697):
 * expert_bounds[e] .. expert_bounds[e+1] delimit, in pair_order, the (token*k + route) pair
 * indices routed to expert e (ascending -- the reference fills them in arbitrary order);
 * tile_bounds counts tiles of tile_m pairs per expert.  All arrays are device int32:
 * expert_bounds and tile_bounds [experts+1], pair_order [tokens*k].
 * --------------------------------------------------------------------------------- */
enum { MFQB_ROUTER_SOFTMAX = 0, MFQB_ROUTER_SIGMOID = 1, MFQB_ROUTER_SQRT_SOFTPLUS = 2,
       MFQB_ROUTER_DELAYED_SOFTMAX = 3 };

int mfqb_moe_topk(const float* logits, int tokens, int experts, int k, int mode, const float* bias,
                  int normalize, float norm_floor, float scale, int32_t* ids, float* weights,
                  mfqb_stream_t stream);
int mfqb_moe_route_plan(const int32_t* ids, int tokens, int k, int experts, int tile_m,
                        int32_t* expert_bounds, int32_t* tile_bounds, int32_t* pair_order,
                        mfqb_stream_t stream);

/* ---------------------------------------------------------------------------------
 * Expert-wise mixed-precision weights ("NINTM" records) and the routed expert matmul.
 *
 * mfqb_nintm_from_blob replaces unpack_nint_moe + initialize_nint_moe_dispatch +
 * to_gpu_nint_moe (cpp_runtime/mfq_decode.cpp:2367-2478, 3249-3381); with an expert range
 * [begin, end) it is the expert-parallel shard of to_cuda_device_moe_expert_slice
 * (cpp_runtime/mfq_decode.cpp:5479-5590): only cohort rows of experts in the range are
 * uploaded; the others are "not held" and their routes produce zeros.
 *
 * mfqb_mul_mat_id replaces NintMoeWeight::forward (cpp_runtime/mfq_decode.cpp:2908-3071):
 *   out[t, r, :] = W[ids[t, r]] . x[src],   src = t (x_per_pair = 0, x is [tokens, k])
 *                                            or the pair t*routes + r (x_per_pair = 1).
 * x bf16, ids device int32 [tokens, routes], out [tokens, routes, out_per_expert] in out_dtype.
 * --------------------------------------------------------------------------------- */
typedef struct mfqb_moe_weight mfqb_moe_weight;

typedef struct mfqb_moe_info {
    int n_experts, out_per_expert, k;
    int expert_begin, expert_end;  /* experts held by this handle */
    int n_pools;
    int device;
    uint64_t payload_bytes;        /* file streams of the held experts */
    uint64_t device_bytes;
} mfqb_moe_info;

int mfqb_nintm_from_blob(const void* blob, uint64_t nbytes, int expert_begin, int expert_end,
                         int device, mfqb_moe_weight** out); /* end < 0: all experts */
int mfqb_moe_info_get(const mfqb_moe_weight* w, mfqb_moe_info* info);
/* bytes of the file streams of one expert (0 if not held): the roofline numerator of a step
 * is the sum over the distinct experts it touches */
int mfqb_moe_expert_bytes(const mfqb_moe_weight* w, int expert, uint64_t* payload_bytes);
int mfqb_moe_weight_free(mfqb_moe_weight* w);
/* [out_per_expert, k] float32/bf16 decode of one held expert (bit-identical to
 * dequantize_expertwise, mfq/quantize/expert_nint.py:597-607) */
int mfqb_moe_dequant_expert(const mfqb_moe_weight* w, int expert, void* out, int out_dtype,
                            mfqb_stream_t stream);
int mfqb_mul_mat_id(const mfqb_moe_weight* w, const void* x_bf16, int x_per_pair, const int32_t* ids,
                    int tokens, int routes, void* out, int out_dtype, mfqb_stream_t stream);

/* SwiGLU split (moe_swiglu_split_cuda, mfq/kernels/cuda/moe.cu:2979-2996; glu.cuh:6-17):
 * rows of gate_up are [gate(F) | up(F)]; hidden = up * gate / (1 + exp(-gate)) in float32,
 * stored as bf16.  Weighted reduce (moe_weighted_reduce_cuda, moe.cu:2957-2977):
 * y[t, :] = sum_r weights[t, r] * expert_out[t, r, :] in float32, routes in order. */
int mfqb_moe_swiglu(const void* gate_up, int in_dtype, int rows, int f, void* hidden_bf16,
                    mfqb_stream_t stream);
int mfqb_moe_weighted_reduce(const void* expert_out, int in_dtype, const float* weights, int tokens,
                             int routes, int h, void* y, int y_dtype, mfqb_stream_t stream);

/* Whole expert FFN (nint_moe_ffn_forward, cpp_runtime/mfq_decode.cpp:3394-3416):
 *   y[t] = sum_r weights[t, r] * down_e( silu(gate_e x[t]) * up_e x[t] ),  e = ids[t, r].
 * gate_up holds [E, 2F, H] (gate rows first), down [E, H, F].  The intermediates live in a
 * per-device library buffer that only ever grows (see mfqb_mul_mat): the first call of a given
 * size must come outside stream capture (inside one it fails with MFQB_ERR_ARG), one warm-up call
 * per batch-size regime should precede a capture, and calls on one device must be ordered by
 * their streams.  mfqb_mul_mat_id with tokens * routes >= n_experts uses a buffer of the same kind. */
int mfqb_moe_ffn(const mfqb_moe_weight* gate_up, const mfqb_moe_weight* down, const void* x_bf16,
                 const int32_t* ids, const float* weights, int tokens, int routes, void* y, int y_dtype,
                 mfqb_stream_t stream);

/* ---------------------------------------------------------------------------------
 * Tensor- / expert-parallel reduction.  Replaces reduce_tensor_parallel_outputs
 * (cpp_runtime/mfq_decode.cpp:9009-9114: float32 ncclAllReduce, or copy-to-primary and add)
 * for the decode-sized vectors of row-parallel linears and expert-parallel FFN partials:
 * a one-shot all-reduce over NVLink peer memory -- every rank stores its vector into every
 * peer (each value paired with the call's number in one 8-byte store), waits (bounded) until
 * its own slots carry that number and adds them in rank order, so all ranks end with
 * bit-identical sums.  The call number lives in device memory: calls may be captured into a
 * CUDA graph and replayed.  One process per GPU; the per-rank buffers are
 * shared with CUDA IPC handles that the caller exchanges (64 bytes each).
 *
 *   create -> handle (send to every peer) -> attach(peer, its handle) for every other rank
 *   -> allreduce ... -> destroy.   All ranks must issue the same sequence of allreduce calls
 * with the same n.  A wait that passes its deadline (default 2 s) sets the status word to
 * MFQB_ERR_TIMEOUT and lets the kernel return; mfqb_comm_status reads it without
 * synchronising.  max_elems <= 4194304 floats, world <= 8.
 *
 * mfqb_mul_mat_allreduce is the row-parallel linear itself (forward_tensor_parallel_flat +
 * reduce, cpp_runtime/mfq_decode.cpp:9137-9207): every rank holds an input-axis slice of the
 * weight (mfqb_weight_from_blob_slice, axis 1) and the matching slice x[m, k_slice]; the
 * product kernel's own epilogue pushes its float32 partial rows to the peers and writes the sum
 * over ranks, y[m, n], on every rank -- one kernel per rank instead of a product, a partial
 * vector in memory and a collective.  It counts as one collective call per activation row in the
 * sequence all ranks must share; n <= max_elems.
 * --------------------------------------------------------------------------------- */
typedef struct mfqb_comm mfqb_comm;
int mfqb_comm_create(int rank, int world, uint64_t max_elems, int device, mfqb_comm** out);
int mfqb_comm_handle(const mfqb_comm* c, void* handle64);
int mfqb_comm_attach(mfqb_comm* c, int peer, const void* handle64);
int mfqb_comm_set_timeout_ms(mfqb_comm* c, int ms);
int mfqb_allreduce_f32(mfqb_comm* c, const float* in, float* out, uint64_t n, mfqb_stream_t stream);
int mfqb_mul_mat_allreduce(const mfqb_weight* w, const void* x_bf16, int m, mfqb_comm* c, void* y, int y_dtype,
                           mfqb_stream_t stream);
/* Recovery after MFQB_ERR_TIMEOUT.  Every rank calls it with none of its collectives in flight;
 * it clears this rank's slots, its device-side call number and its status word.  The ranks must
 * then synchronise on the host (a barrier of the caller's process group) before the next
 * collective.  No counterpart in the reference (NCCL errors there end the process,
 * cpp_runtime/mfq_decode.cpp:63-70). */
int mfqb_comm_reset(mfqb_comm* c);
/* Test hook: sets the device-side call number, e.g. just below the 32-bit wrap (every rank the same value). */
int mfqb_comm_debug_set_seq(mfqb_comm* c, unsigned seq);
int mfqb_comm_status(const mfqb_comm* c, int* status);
int mfqb_comm_destroy(mfqb_comm* c);

/* Expert FFN that allocates nothing.  (No counterpart in the reference runtime, whose FFN takes
 * its workspaces from the libtorch caching allocator.)
 *
 * Same result as mfqb_moe_ffn, for callers that are not allowed to allocate device memory at the
 * point of the call: code running while a stream is being captured into a graph, a serving loop
 * that has handed all free HBM to its KV cache and must not fragment it, or a host process whose
 * allocator hooks forbid cudaMalloc on the hot path.  The three intermediates (gate/up
 * products, the SwiGLU activation, the down products) go into one fixed array of
 * MFQB_STATIC_SCRATCH_BYTES that is part of the library image; every GPU that loads the library
 * holds that much memory until the process exits.
 *
 *  - 64 KiB of counters + tokens * routes * (2F*4 + F*4 + H*4) bytes (rounded up a little; plus the
 *    route plan and the quantised planes for batches that take the tiled kernels) must fit; a larger
 *    call is rejected with MFQB_ERR_ARG and a message giving both numbers -- use mfqb_moe_ffn then.
 *  - The first call on a device looks the array's device address up (once per device, with that
 *    device current), and the first launch of each kernel variant (the single-row kernel for few
 *    tokens, the tiled kernels per tile size for larger batches) sets its function attributes and
 *    makes the driver load its code.  Make one call per batch-size regime you will use before any
 *    stream capture; after that the call can be recorded into a graph.
 *  - All calls share the one array and it keeps the previous call's contents; each call clears
 *    the counters at its start first (everything else is written before it is read).  Two calls whose device work overlaps (different streams, or
 *    different host threads) race on it: serialise them.
 *  - It calls no cudaMalloc / cudaFree and no library routine that allocates. */
#define MFQB_STATIC_SCRATCH_BYTES (8u << 20)
int mfqb_moe_ffn_static(const mfqb_moe_weight* gate_up, const mfqb_moe_weight* down, const void* x_bf16,
                        const int32_t* ids, const float* weights, int tokens, int routes, void* y,
                        int y_dtype, mfqb_stream_t stream);

/* ---------------------------------------------------------------------------------
 * Dense decoder step: the runtime layer around the packed-weight products.  Stands in for
 * QuantLinear / FFN / FullBlock::forward / Model::next_token of the reference runtime
 * (cpp_runtime/mfq_decode.cpp:9116-9407, 10456-10602, 12210-12400, 13993-14145) for one model
 * family: Llama-shaped blocks (RMSNorm, rotary embedding with the halves convention, grouped-query
 * attention over a bf16 KV cache, SwiGLU FFN), greedy decoding.  The projections are weight handles
 * of this library, borrowed for the decoder's lifetime; q|k|v and gate|up are single fused handles.
 * With world > 1 every rank holds n_q/world query heads, n_kv/world KV heads (and their cache),
 * ffn/world FFN columns and a slice of the vocabulary; o_proj and down_proj hold the matching input
 * slices and end in a sum over the ranks of `comm`.
 * --------------------------------------------------------------------------------- */
typedef struct mfqb_decoder mfqb_decoder;
typedef struct mfqb_decoder_config {
    int hidden, n_q_heads, n_kv_heads, head_dim; /* head_dim must be 128; hidden = n_q_heads * 128 */
    int ffn, vocab, layers;
    int max_ctx, max_batch;
    float rope_theta, rms_eps;
} mfqb_decoder_config;
int mfqb_decoder_create(const mfqb_decoder_config* cfg, int rank, int world, mfqb_comm* comm, int device,
                        mfqb_decoder** out);
/* This rank's shapes: qkv [(n_q + 2 n_kv)/world * 128, hidden] (query rows, key rows, value rows);
 * o [hidden, n_q/world * 128]; gate_up [2 * ffn/world, hidden] in 16-row blocks that
 * alternate gate rows and up rows (the layout of mfqb_mul_mat_glu); down [hidden, ffn/world];
 * ffn/world must be a multiple of 16. */
int mfqb_decoder_set_layer(mfqb_decoder* d, int layer, const mfqb_weight* qkv, const mfqb_weight* o,
                           const mfqb_weight* gate_up, const mfqb_weight* down);
/* lm_head: rows [begin, begin + rows) of the vocabulary (mfqb_decoder_vocab_shard) x hidden;
 * embedding: bf16 [vocab, hidden] in device memory (replicated). */
int mfqb_decoder_vocab_shard(const mfqb_decoder* d, int* begin, int* rows);
int mfqb_decoder_set_head(mfqb_decoder* d, const mfqb_weight* lm_head, const void* embedding_bf16);
/* Fills the first ctx_len cache positions of every sequence with seeded values of unit scale (a
 * stand-in for the prefill pass, which is outside this path) and sets every position to ctx_len. */
int mfqb_decoder_fill_cache(mfqb_decoder* d, int ctx_len, unsigned seed, mfqb_stream_t stream);
/* One greedy step for `batch` sequences: ids_in [batch] -> ids_out [batch] (device int32), positions
 * advance by one.  All device work goes to `stream`; the call can be captured in a CUDA graph after
 * one warm-up call (library scratch, see mfqb_mul_mat). */
int mfqb_decoder_step(mfqb_decoder* d, const int32_t* ids_in, int batch, int32_t* ids_out,
                      mfqb_stream_t stream);
/* Parity hooks: one block on a given residual stream (float32 [rows, hidden] in and out, cache
 * positions as currently set, the step's key/value rows are written); and a read-back of one
 * sequence's cache rows, which = 0 keys / 1 values, as bf16 [n_kv/world][ctx][128]. */
int mfqb_decoder_layer(mfqb_decoder* d, int layer, const float* h_in, int rows, float* h_out,
                       mfqb_stream_t stream);
int mfqb_decoder_read_cache(const mfqb_decoder* d, int layer, int row, int which, int ctx, void* out_bf16,
                            mfqb_stream_t stream);
/* The logits of the last mfqb_decoder_step, this rank's vocabulary rows: out [rows, shard rows] float32. */
int mfqb_decoder_read_logits(const mfqb_decoder* d, int rows, float* out, mfqb_stream_t stream);
int mfqb_decoder_free(mfqb_decoder* d);

/* ---------------------------------------------------------------------------------
 * Host-side self-check of the device layout (no GPU): packs the blob into the device
 * format, reads every code and scale field back through the same accessors the kernels
 * use, and reports the number of mismatches against the file streams.
 * --------------------------------------------------------------------------------- */
int mfqb_selfcheck_layout(const char* dtype, const void* blob, uint64_t nbytes,
                          uint64_t* mismatches);

#ifdef __cplusplus
}
#endif
#endif /* MFQB200_H */
