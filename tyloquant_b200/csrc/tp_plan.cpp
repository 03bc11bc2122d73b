// Tensor-parallel slice planner: same boundaries and the same rejections as
// plan_tensor_parallel_slices / validate_tensor_parallel_slices
// (cpp_runtime/tensor_parallel.h:23-118) and tensor_parallel_granularity
// (cpp_runtime/mfq_decode.cpp:9445-9461).
#include <algorithm>
#include <cmath>

#include "common.h"

using namespace mfqb;

extern "C" {
#pragma GCC visibility push(default)

int mfqb_tp_plan(int64_t extent, int64_t granularity, int n_devices, const double* weights, int64_t* begins,
                 int64_t* ends) {
    return guarded([&] {
        if (!begins || !ends) fail(MFQB_ERR_ARG, "mfqb_tp_plan: null output");
        if (extent <= 0) fail(MFQB_ERR_ARG, "tensor-parallel extent must be positive");
        if (granularity <= 0) fail(MFQB_ERR_ARG, "tensor-parallel granularity must be positive");
        if (n_devices <= 0) fail(MFQB_ERR_ARG, "tensor-parallel device list must not be empty");
        if (extent < (int64_t)n_devices * granularity)
            fail(MFQB_ERR_ARG, "tensor-parallel extent is too small for the device count");
        std::vector<double> share((size_t)n_devices, 1.0 / (double)n_devices);
        if (weights) {
            double sum = 0.0;
            for (int i = 0; i < n_devices; ++i) {
                if (!std::isfinite(weights[i]) || weights[i] <= 0.0)
                    fail(MFQB_ERR_ARG, "tensor-parallel split weights must be finite and positive");
                sum += weights[i];
            }
            for (int i = 0; i < n_devices; ++i) share[i] = weights[i] / sum;
        }
        std::vector<int64_t> edge((size_t)n_devices + 1, 0);
        edge[n_devices] = extent;
        double cumulative = 0.0;
        for (int i = 1; i < n_devices; ++i) {
            cumulative += share[i - 1];
            const double target = cumulative * (double)extent;
            const int64_t snapped = (int64_t)std::llround(target / (double)granularity) * granularity;
            const int64_t lowest = edge[i - 1] + granularity;
            const int64_t highest = extent - (int64_t)(n_devices - i) * granularity;
            edge[i] = std::min(std::max(snapped, lowest), highest);
        }
        for (int i = 0; i < n_devices; ++i) {
            begins[i] = edge[i];
            ends[i] = edge[i + 1];
        }
    });
}

int mfqb_tp_validate(int64_t extent, int64_t granularity, int n_slices, const int64_t* begins, const int64_t* ends) {
    return guarded([&] {
        if (!begins || !ends || n_slices <= 0 || begins[0] != 0 || ends[n_slices - 1] != extent)
            fail(MFQB_ERR_ARG, "tensor-parallel slices do not cover the full extent");
        if (granularity <= 0) fail(MFQB_ERR_ARG, "tensor-parallel granularity must be positive");
        for (int i = 0; i < n_slices; ++i) {
            if (begins[i] >= ends[i]) fail(MFQB_ERR_ARG, "tensor-parallel slice must not be empty");
            if (i > 0 && ends[i - 1] != begins[i]) fail(MFQB_ERR_ARG, "tensor-parallel slices must be contiguous");
            if (i + 1 < n_slices && (begins[i] % granularity != 0 || ends[i] % granularity != 0))
                fail(MFQB_ERR_ARG, "interior tensor-parallel boundaries are misaligned");
        }
    });
}

int mfqb_tp_granularity(int64_t extent, int64_t preferred, int n_devices, int64_t* out) {
    return guarded([&] {
        if (!out || n_devices <= 0 || extent <= 0) fail(MFQB_ERR_ARG, "mfqb_tp_granularity: bad argument");
        int64_t g = std::max<int64_t>(1, std::min<int64_t>(preferred, extent / n_devices));
        while (g > 1 && extent < (int64_t)n_devices * g) g /= 2;
        *out = std::max<int64_t>(1, g);
    });
}

#pragma GCC visibility pop
}  // extern "C"
