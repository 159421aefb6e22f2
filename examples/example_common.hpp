// Shared helpers of the example drivers: positional command line of the reference examples
// (verify 0/1, init 0 none | 1 integers | 2 decimals, time 0/1, then shapes), the perf line
// "Perf: <ms> ms, <tflops> TFlops, <GB/s> GB/s, <type string>", and row/column-major host descriptors.
#pragma once
#include <cstdio>
#include <cstdlib>
#include <iostream>
#include <string>
#include <type_traits>
#include <vector>

#include "ck/ck.hpp"
#include "ck/library/host_tensor/host_tensor.hpp"
#include "ck/tensor_operation/gpu/device/tensor_layout.hpp"

namespace example {

struct RunFlags
{
    bool do_verification = true;
    int init_method      = 1;
    bool time_kernel     = false;
};

// Reads argv[1..3] when present; returns the index of the first shape argument.
inline int parse_flags(int argc, char* argv[], RunFlags& f)
{
    if(argc >= 4)
    {
        f.do_verification = std::stoi(argv[1]) != 0;
        f.init_method     = std::stoi(argv[2]);
        f.time_kernel     = std::stoi(argv[3]) != 0;
        return 4;
    }
    return 1;
}

inline void usage_and_exit(const char* shapes)
{
    std::printf("arg1: verification (0=no, 1=yes)\n");
    std::printf("arg2: initialization (0=no init, 1=integer value, 2=decimal value)\n");
    std::printf("arg3: time kernel (0=no, 1=yes)\n");
    std::printf("%s\n", shapes);
    std::exit(0);
}

template <typename Layout>
HostTensorDescriptor matrix_descriptor(std::size_t row, std::size_t col, std::size_t stride, Layout)
{
    if(std::is_same<Layout, ck::tensor_layout::gemm::RowMajor>::value)
        return HostTensorDescriptor(std::vector<std::size_t>{row, col}, std::vector<std::size_t>{stride, 1});
    return HostTensorDescriptor(std::vector<std::size_t>{row, col}, std::vector<std::size_t>{1, stride});
}

inline void print_perf(float ave_time_ms, std::size_t flop, std::size_t num_btype, const std::string& type_string)
{
    const float tflops     = static_cast<float>(flop) / 1.E9 / ave_time_ms;
    const float gb_per_sec = num_btype / 1.E6 / ave_time_ms;
    std::cout << "Perf: " << ave_time_ms << " ms, " << tflops << " TFlops, " << gb_per_sec << " GB/s, " << type_string
              << std::endl;
}

} // namespace example
