// A client of the instance factory in the style of the reference's client_example/01_gemm/gemm.cpp: it includes only
// the device-operation interface and the instance list, walks the list, times every instance that supports the
// problem and runs the best one again.  The only change against the reference client is the allocator behind
// SimpleDeviceMem (the library's C ABI instead of hipMalloc).
//   usage: client_gemm [M N K StrideA StrideB StrideC]
#include <cstdio>
#include <cstdlib>
#include <iomanip>
#include <iostream>
#include <string>
#include <vector>

#include "ck/ck.hpp"
#include "ck/library/tensor_operation_instance/gpu/gemm.hpp"
#include "ck/tensor_operation/gpu/device/device_gemm.hpp"
#include "ck/tensor_operation/gpu/device/tensor_layout.hpp"
#include "ck/tensor_operation/gpu/element/element_wise_operation.hpp"

using F16 = ck::half_t;
using Row = ck::tensor_layout::gemm::RowMajor;
using Col = ck::tensor_layout::gemm::ColumnMajor;
using PassThrough = ck::tensor_operation::element_wise::PassThrough;

using ADataType = F16;
using BDataType = F16;
using CDataType = F16;
using ALayout   = Row;
using BLayout   = Col;
using CLayout   = Row;

struct SimpleDeviceMem
{
    SimpleDeviceMem() = delete;
    explicit SimpleDeviceMem(std::size_t mem_size) : p_mem_{} { (void)ckb_malloc(&p_mem_, mem_size); }
    void* GetDeviceBuffer() { return p_mem_; }
    ~SimpleDeviceMem() { (void)ckb_free(p_mem_); }
    void* p_mem_;
};

template <typename Layout>
std::size_t matrix_space_size(std::size_t rows, std::size_t cols, std::size_t stride, Layout)
{
    return std::is_same<Layout, Row>::value ? (rows - 1) * stride + cols : (cols - 1) * stride + rows;
}

int main(int argc, char* argv[])
{
    ck::index_t M = 3840, N = 4096, K = 4096, StrideA = 4096, StrideB = 4096, StrideC = 4096;
    if(argc == 7)
    {
        M = std::stoi(argv[1]), N = std::stoi(argv[2]), K = std::stoi(argv[3]);
        StrideA = std::stoi(argv[4]), StrideB = std::stoi(argv[5]), StrideC = std::stoi(argv[6]);
    }
    else if(argc != 1)
    {
        std::printf("arg1 to 6: M, N, K, StrideA, StrideB, StrideC\n");
        return 0;
    }

    SimpleDeviceMem a_device_buf(sizeof(ADataType) * matrix_space_size(M, K, StrideA, ALayout{}));
    SimpleDeviceMem b_device_buf(sizeof(BDataType) * matrix_space_size(K, N, StrideB, BLayout{}));
    SimpleDeviceMem c_device_buf(sizeof(CDataType) * matrix_space_size(M, N, StrideC, CLayout{}));

    using DeviceOp = ck::tensor_operation::device::DeviceGemm<ALayout, BLayout, CLayout, ADataType, BDataType, CDataType,
                                                              PassThrough, PassThrough, PassThrough>;
    const auto op_ptrs =
        ck::tensor_operation::device::instance::DeviceOperationInstanceFactory<DeviceOp>::GetInstances();
    std::cout << "found " << op_ptrs.size() << " instances" << std::endl;

    auto make_argument = [&](const auto& op_ptr) {
        return op_ptr->MakeArgumentPointer(a_device_buf.GetDeviceBuffer(), b_device_buf.GetDeviceBuffer(),
                                           c_device_buf.GetDeviceBuffer(), M, N, K, StrideA, StrideB, StrideC,
                                           PassThrough{}, PassThrough{}, PassThrough{});
    };

    std::string best_op_name;
    int best_op_id        = -1;
    float best_ave_time   = 0;
    float best_tflops     = 0;
    float best_gb_per_sec = 0;
    std::cout << "Run all instances and do timing" << std::endl;
    for(std::size_t i = 0; i < op_ptrs.size(); ++i)
    {
        auto& op_ptr              = op_ptrs[i];
        auto argument_ptr         = make_argument(op_ptr);
        auto invoker_ptr          = op_ptr->MakeInvokerPointer();
        const std::string op_name = op_ptr->GetTypeString();
        if(!op_ptr->IsSupportedArgument(argument_ptr.get()))
        {
            std::cout << op_name << " does not support this problem" << std::endl;
            continue;
        }
        const float ave_time        = invoker_ptr->Run(argument_ptr.get(), StreamConfig{nullptr, true});
        const std::size_t flop      = std::size_t(2) * M * N * K;
        const std::size_t num_btype = sizeof(ADataType) * M * K + sizeof(BDataType) * K * N + sizeof(CDataType) * M * N;
        const float tflops          = static_cast<float>(flop) / 1.E9 / ave_time;
        const float gb_per_sec      = num_btype / 1.E6 / ave_time;
        std::cout << "Perf: " << std::setw(10) << ave_time << " ms, " << tflops << " TFlops, " << gb_per_sec << " GB/s, "
                  << op_name << std::endl;
        if(tflops > best_tflops)
        {
            best_op_id      = static_cast<int>(i);
            best_op_name    = op_name;
            best_tflops     = tflops;
            best_ave_time   = ave_time;
            best_gb_per_sec = gb_per_sec;
        }
    }
    if(best_op_id < 0)
    {
        std::cout << "no instance supports this problem" << std::endl;
        return 1;
    }
    std::cout << "Best Perf: " << best_ave_time << " ms, " << best_tflops << " TFlops, " << best_gb_per_sec << " GB/s, "
              << best_op_name << std::endl;

    auto& op_ptr = op_ptrs[best_op_id];
    std::cout << "Run the best instance without timing: " << op_ptr->GetTypeString() << std::endl;
    auto argument_ptr = make_argument(op_ptr);
    auto invoker_ptr  = op_ptr->MakeInvokerPointer();
    if(op_ptr->IsSupportedArgument(argument_ptr.get()))
        invoker_ptr->Run(argument_ptr.get(), StreamConfig{nullptr, false});
    if(ckb_device_synchronize() != CKB_OK)
        return 1;
    std::cout << "Done" << std::endl;
    return 0;
}
