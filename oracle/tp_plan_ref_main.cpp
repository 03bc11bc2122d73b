// Test infrastructure: command-line driver around the reference's own slice planner header
// (cpp_runtime/tensor_parallel.h, compiled in place from the reference tree, never copied).
//   tp_plan_ref <extent> <granularity> <n_devices> [weights...]
// prints "begin end" per device, or "throw: <message>" when the planner or its validator throws.
#include <cstdlib>
#include <iostream>
#include <vector>

#include "tensor_parallel.h"

int main(int argc, char** argv) {
    if (argc < 4) return 2;
    const long long extent = std::atoll(argv[1]), gran = std::atoll(argv[2]);
    const int n = std::atoi(argv[3]);
    std::vector<int> devices;
    for (int i = 0; i < n; ++i) devices.push_back(i);
    std::vector<double> weights;
    for (int i = 4; i < argc; ++i) weights.push_back(std::atof(argv[i]));
    try {
        const auto slices = mfq::plan_tensor_parallel_slices(extent, gran, devices, weights);
        for (const auto& s : slices) std::cout << s.begin << " " << s.end << "\n";
        try {
            mfq::validate_tensor_parallel_slices(slices, extent, gran);
            std::cout << "valid\n";
        } catch (const std::exception& e) {
            std::cout << "invalid: " << e.what() << "\n";
        }
    } catch (const std::exception& e) {
        std::cout << "throw: " << e.what() << "\n";
    }
    return 0;
}
