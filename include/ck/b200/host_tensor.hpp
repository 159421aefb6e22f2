// Host-side tensors, generators and device buffers used by example / profiler style drivers.
// Same names and member functions as the reference's host_tensor library
// (library/include/ck/library/host_tensor/host_tensor.hpp:74-369, host_tensor_generator.hpp:11-153,
// device_memory.hpp:17-40); device memory goes through the C ABI of ckb200.h.
#pragma once
#include <algorithm>
#include <array>
#include <cmath>
#include <cstdlib>
#include <functional>
#include <iostream>
#include <numeric>
#include <stdexcept>
#include <string>
#include <thread>
#include <tuple>
#include <utility>
#include <vector>

#include "ck/b200/core.hpp"
#include "ckb200.h"

// Lengths + strides of a host tensor (element strides).
struct HostTensorDescriptor
{
    HostTensorDescriptor() = delete;

    template <typename X>
    HostTensorDescriptor(const std::vector<X>& lens) : mLens(lens.begin(), lens.end())
    {
        CalculateStrides();
    }
    template <typename X>
    HostTensorDescriptor(std::initializer_list<X> lens) : mLens(lens.begin(), lens.end())
    {
        CalculateStrides();
    }
    template <typename X, typename Y>
    HostTensorDescriptor(const std::vector<X>& lens, const std::vector<Y>& strides)
        : mLens(lens.begin(), lens.end()), mStrides(strides.begin(), strides.end())
    {
    }

    // packed, last dimension fastest
    void CalculateStrides()
    {
        mStrides.assign(mLens.size(), 1);
        for(std::size_t i = mLens.size(); i-- > 1;)
            mStrides[i - 1] = mStrides[i] * mLens[i];
    }
    std::size_t GetNumOfDimension() const { return mLens.size(); }
    std::size_t GetElementSize() const
    {
        return std::accumulate(mLens.begin(), mLens.end(), std::size_t{1}, std::multiplies<std::size_t>());
    }
    // library/src/host_tensor/host_tensor.cpp:26-35: 1 + sum (len - 1) * stride
    std::size_t GetElementSpace() const
    {
        std::size_t space = 1;
        for(std::size_t i = 0; i < mLens.size(); ++i)
            space += (mLens[i] - 1) * mStrides[i];
        return space;
    }
    const std::vector<std::size_t>& GetLengths() const { return mLens; }
    const std::vector<std::size_t>& GetStrides() const { return mStrides; }

    template <typename... Is>
    std::size_t GetOffsetFromMultiIndex(Is... is) const
    {
        const std::size_t idx[] = {static_cast<std::size_t>(is)...};
        std::size_t off         = 0;
        for(std::size_t i = 0; i < sizeof...(Is); ++i)
            off += idx[i] * mStrides[i];
        return off;
    }
    std::size_t GetOffsetFromMultiIndex(const std::vector<std::size_t>& idx) const
    {
        return std::inner_product(idx.begin(), idx.end(), mStrides.begin(), std::size_t{0});
    }

    friend std::ostream& operator<<(std::ostream& os, const HostTensorDescriptor& d)
    {
        os << "dim " << d.GetNumOfDimension() << ", lengths {";
        for(std::size_t i = 0; i < d.mLens.size(); ++i)
            os << (i ? ", " : "") << d.mLens[i];
        os << "}, strides {";
        for(std::size_t i = 0; i < d.mStrides.size(); ++i)
            os << (i ? ", " : "") << d.mStrides[i];
        return os << "}";
    }

    private:
    std::vector<std::size_t> mLens;
    std::vector<std::size_t> mStrides;
};

// host_tensor.hpp:142-194: the flattened index space is cut into equal contiguous chunks, one
// std::thread per chunk.
template <typename F, typename... Xs>
struct ParallelTensorFunctor
{
    static constexpr std::size_t NDIM = sizeof...(Xs);
    F mF;
    std::array<std::size_t, NDIM> mLens;
    std::array<std::size_t, NDIM> mStrides;
    std::size_t mN1d;

    ParallelTensorFunctor(F f, Xs... xs) : mF(f), mLens({static_cast<std::size_t>(xs)...})
    {
        mStrides[NDIM - 1] = 1;
        for(std::size_t i = NDIM - 1; i > 0; --i)
            mStrides[i - 1] = mStrides[i] * mLens[i];
        mN1d = mStrides[0] * mLens[0];
    }
    std::array<std::size_t, NDIM> GetNdIndices(std::size_t i) const
    {
        std::array<std::size_t, NDIM> idx;
        for(std::size_t d = 0; d < NDIM; ++d)
        {
            idx[d] = i / mStrides[d];
            i -= idx[d] * mStrides[d];
        }
        return idx;
    }
    void operator()(std::size_t num_thread = 1) const
    {
        num_thread                        = std::max<std::size_t>(num_thread, 1);
        const std::size_t work_per_thread = (mN1d + num_thread - 1) / num_thread;
        std::vector<std::thread> threads;
        for(std::size_t it = 0; it < num_thread; ++it)
        {
            const std::size_t begin = it * work_per_thread;
            const std::size_t end   = std::min((it + 1) * work_per_thread, mN1d);
            if(begin >= end)
                break;
            threads.emplace_back([this, begin, end] {
                for(std::size_t iw = begin; iw < end; ++iw)
                    std::apply(mF, GetNdIndices(iw));
            });
        }
        for(auto& t : threads)
            t.join();
    }
};
template <typename F, typename... Xs>
auto make_ParallelTensorFunctor(F f, Xs... xs)
{
    return ParallelTensorFunctor<F, Xs...>(f, xs...);
}

template <typename T>
struct Tensor
{
    template <typename X>
    Tensor(std::initializer_list<X> lens) : mDesc(lens), mData(mDesc.GetElementSpace())
    {
    }
    template <typename X>
    Tensor(std::vector<X> lens) : mDesc(lens), mData(mDesc.GetElementSpace())
    {
    }
    template <typename X, typename Y>
    Tensor(std::vector<X> lens, std::vector<Y> strides) : mDesc(lens, strides), mData(mDesc.GetElementSpace())
    {
    }
    Tensor(const HostTensorDescriptor& desc) : mDesc(desc), mData(mDesc.GetElementSpace()) {}

    template <typename OutT>
    Tensor<OutT> CopyAsType() const
    {
        Tensor<OutT> ret(mDesc);
        for(std::size_t i = 0; i < mData.size(); ++i)
            ret.mData[i] = static_cast<OutT>(mData[i]);
        return ret;
    }

    template <typename F>
    void ForEach(F&& f)
    {
        std::vector<std::size_t> idx(mDesc.GetNumOfDimension(), 0);
        for_each_rec(f, idx, 0);
    }

    // value at every multi-index = g(indices...), filled with num_thread threads
    template <typename G>
    void GenerateTensorValue(G g, std::size_t num_thread = 1)
    {
        const auto& L = mDesc.GetLengths();
        switch(mDesc.GetNumOfDimension())
        {
        case 1: make_ParallelTensorFunctor([&](auto i) { (*this)(i) = g(i); }, L[0])(num_thread); break;
        case 2:
            make_ParallelTensorFunctor([&](auto i, auto j) { (*this)(i, j) = g(i, j); }, L[0], L[1])(num_thread);
            break;
        case 3:
            make_ParallelTensorFunctor([&](auto i, auto j, auto k) { (*this)(i, j, k) = g(i, j, k); }, L[0], L[1],
                                       L[2])(num_thread);
            break;
        case 4:
            make_ParallelTensorFunctor([&](auto i, auto j, auto k, auto l) { (*this)(i, j, k, l) = g(i, j, k, l); },
                                       L[0], L[1], L[2], L[3])(num_thread);
            break;
        case 5:
            make_ParallelTensorFunctor(
                [&](auto i, auto j, auto k, auto l, auto m) { (*this)(i, j, k, l, m) = g(i, j, k, l, m); }, L[0], L[1],
                L[2], L[3], L[4])(num_thread);
            break;
        default: throw std::runtime_error("unspported dimension");
        }
    }

    template <typename... Is>
    T& operator()(Is... is)
    {
        return mData[mDesc.GetOffsetFromMultiIndex(is...)];
    }
    template <typename... Is>
    const T& operator()(Is... is) const
    {
        return mData[mDesc.GetOffsetFromMultiIndex(is...)];
    }
    T& operator()(const std::vector<std::size_t>& idx) { return mData[mDesc.GetOffsetFromMultiIndex(idx)]; }
    const T& operator()(const std::vector<std::size_t>& idx) const
    {
        return mData[mDesc.GetOffsetFromMultiIndex(idx)];
    }

    typename std::vector<T>::iterator begin() { return mData.begin(); }
    typename std::vector<T>::iterator end() { return mData.end(); }
    typename std::vector<T>::const_iterator begin() const { return mData.begin(); }
    typename std::vector<T>::const_iterator end() const { return mData.end(); }

    HostTensorDescriptor mDesc;
    std::vector<T> mData;

    private:
    template <typename F>
    void for_each_rec(F& f, std::vector<std::size_t>& idx, std::size_t rank)
    {
        if(rank == mDesc.GetNumOfDimension())
        {
            f(*this, idx);
            return;
        }
        for(std::size_t i = 0; i < mDesc.GetLengths()[rank]; ++i)
        {
            idx[rank] = i;
            for_each_rec(f, idx, rank + 1);
        }
    }
};

// ---- generators (host_tensor_generator.hpp) -------------------------------------------------------
template <typename T>
struct GeneratorTensor_0
{
    template <typename... Is>
    T operator()(Is...)
    {
        return T{0};
    }
};
template <typename T>
struct GeneratorTensor_1
{
    int value = 1;
    template <typename... Is>
    T operator()(Is...)
    {
        return ck::type_convert<T>(static_cast<float>(value));
    }
};
// integers in [min_value, max_value - 1] from std::rand() (host_tensor_generator.hpp:58-95)
template <typename T>
struct GeneratorTensor_2
{
    int min_value = 0;
    int max_value = 1;
    template <typename... Is>
    T operator()(Is...)
    {
        return ck::type_convert<T>(static_cast<float>((std::rand() % (max_value - min_value)) + min_value));
    }
};
// uniform reals in [min_value, max_value] from std::rand() (host_tensor_generator.hpp:98-127)
template <typename T>
struct GeneratorTensor_3
{
    float min_value = 0;
    float max_value = 1;
    template <typename... Is>
    T operator()(Is...)
    {
        const float tmp = float(std::rand()) / float(RAND_MAX);
        return ck::type_convert<T>(min_value + tmp * (max_value - min_value));
    }
};
template <ck::index_t Dim>
struct GeneratorTensor_Sequential
{
    template <typename... Ts>
    float operator()(Ts... Xs) const
    {
        std::array<ck::index_t, sizeof...(Ts)> dims = {{static_cast<ck::index_t>(Xs)...}};
        return dims[Dim];
    }
};

// ---- device buffer (device_memory.hpp:17-40, device_memory.cpp:7-28) ------------------------------
struct DeviceMem
{
    DeviceMem() = delete;
    DeviceMem(std::size_t mem_size) : mMemSize(mem_size)
    {
        if(ckb_malloc(&mpDeviceBuf, mMemSize ? mMemSize : 1) != CKB_OK)
            throw std::runtime_error(ckb_last_error());
    }
    DeviceMem(const DeviceMem&) = delete;
    DeviceMem& operator=(const DeviceMem&) = delete;
    void* GetDeviceBuffer() { return mpDeviceBuf; }
    std::size_t GetBufferSize() { return mMemSize; }
    void ToDevice(const void* p)
    {
        if(ckb_memcpy_h2d(mpDeviceBuf, p, mMemSize) != CKB_OK)
            throw std::runtime_error(ckb_last_error());
    }
    void FromDevice(void* p)
    {
        if(ckb_memcpy_d2h(p, mpDeviceBuf, mMemSize) != CKB_OK)
            throw std::runtime_error(ckb_last_error());
    }
    void SetZero()
    {
        if(ckb_memset(mpDeviceBuf, 0, mMemSize) != CKB_OK)
            throw std::runtime_error(ckb_last_error());
    }
    ~DeviceMem() { ckb_free(mpDeviceBuf); }

    void* mpDeviceBuf = nullptr;
    std::size_t mMemSize;
};
