// qmlp::Tensor (src_cpp/include/qmlp/tensor.h:22-253): a strided view of device memory that either refers to memory of
// the caller or owns a cudaMalloc'ed block. Sizes and strides are int32 in elements, as in the reference; view() hands
// the tensor to the C ABI.
#pragma once
#include <cstdint>
#include <memory>
#include <random>
#include <vector>

#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "errors.h"

namespace qmlp {

class Tensor {
public:
    enum Precision { FLOAT, HALF, DOUBLE, _NUM_PRECISION_ };
    enum Usage { INFERENCE, GRADIENTS };
    static int bytesPerEntryOf(Precision p) { return p == FLOAT ? 4 : p == HALF ? 2 : 8; }

    // an undefined tensor (defined() == false)
    Tensor() = default;

    // Non-owning: the caller keeps `data` alive (tensor.h:72-85).
    Tensor(void* data, Precision precision, const std::vector<int32_t>& sizes, const std::vector<int32_t>& strides)
        : data_(data), precision_(precision), sizes_(sizes), strides_(strides)
    {
        if (sizes.empty() || sizes.size() != strides.size()) throw std::runtime_error("sizes and strides must have the same, non-zero length");
    }

    // Owning, contiguous (tensor.h:92, src_cpp/src/tensor.cpp:18-37).
    Tensor(Precision precision, const std::vector<int32_t>& sizes) : precision_(precision), sizes_(sizes)
    {
        if (sizes.empty()) throw std::runtime_error("sizes must not be empty");
        strides_.resize(sizes.size());
        int64_t stride = 1;
        for (int i = static_cast<int>(sizes.size()) - 1; i >= 0; --i) {
            strides_[i] = static_cast<int32_t>(stride);
            stride *= sizes[i];
        }
        void* p = nullptr;
        const size_t bytes = static_cast<size_t>(stride) * bytesPerEntryOf(precision);
        if (bytes > 0) {
            const cudaError_t e = cudaMalloc(&p, bytes);
            if (e != cudaSuccess) throw std::runtime_error(std::string("cudaMalloc: ") + cudaGetErrorString(e));
        }
        owned_ = std::shared_ptr<void>(p, [](void* q) { if (q) cudaFree(q); });
        data_ = p;
    }

    bool defined() const { return !sizes_.empty(); }
    Precision precision() const { return precision_; }
    int bytesPerEntry() const { return bytesPerEntryOf(precision_); }
    int ndim() const { return static_cast<int>(sizes_.size()); }
    const std::vector<int32_t>& sizes() const { return sizes_; }
    int32_t size(int dim) const { return sizes_.at(dim); }
    const std::vector<int32_t>& strides() const { return strides_; }
    int32_t stride(int dim) const { return strides_.at(dim); }
    int64_t numel() const
    {
        int64_t n = defined() ? 1 : 0;
        for (int32_t s : sizes_) n *= s;
        return n;
    }
    // bytes from the first to the last addressed entry (tensor.h:133-140)
    int64_t numBytes() const
    {
        if (numel() == 0) return 0;
        int64_t last = 0;
        for (int i = 0; i < ndim(); ++i) last += static_cast<int64_t>(strides_[i]) * (sizes_[i] - 1);
        return (last + 1) * bytesPerEntry();
    }
    const void* rawPtr() const { return data_; }
    void* rawPtr() { return data_; }
    template <typename T> const T* dataPtr() const { assertType<T>(); return static_cast<const T*>(data_); }
    template <typename T> T* dataPtr() { assertType<T>(); return static_cast<T*>(data_); }

    void zero_()
    {
        if (numBytes() == 0) return;
        const cudaError_t e = cudaMemset(data_, 0, static_cast<size_t>(numBytes()));
        if (e != cudaSuccess) throw std::runtime_error(std::string("cudaMemset: ") + cudaGetErrorString(e));
    }
    // uniform random entries from a host generator, uploaded (tensor.h:203-218)
    template <typename RNG> void rand_(float a, float b, RNG& rng)
    {
        std::uniform_real_distribution<float> distr(a, b);
        const int64_t n = numel();
        cudaError_t e = cudaSuccess;
        if (precision_ == FLOAT) {
            std::vector<float> host(static_cast<size_t>(n));
            for (auto& v : host) v = distr(rng);
            e = cudaMemcpy(data_, host.data(), sizeof(float) * host.size(), cudaMemcpyHostToDevice);
        } else if (precision_ == HALF) {
            std::vector<__half> host(static_cast<size_t>(n));
            for (auto& v : host) v = __float2half(distr(rng));
            e = cudaMemcpy(data_, host.data(), sizeof(__half) * host.size(), cudaMemcpyHostToDevice);
        } else {
            throw std::runtime_error("rand_ supports float and half tensors");
        }
        if (e != cudaSuccess) throw std::runtime_error(std::string("cudaMemcpy: ") + cudaGetErrorString(e));
    }
    void copy_(const Tensor& src) { copyAsync_(src, nullptr); cudaStreamSynchronize(nullptr); }
    void copyAsync_(const Tensor& src, cudaStream_t stream)
    {
        if (src.precision_ != precision_ || src.sizes_ != sizes_ || src.strides_ != strides_)
            throw std::runtime_error("copy_ needs tensors of the same precision, sizes and strides");
        const cudaError_t e = cudaMemcpyAsync(data_, src.data_, static_cast<size_t>(numBytes()), cudaMemcpyDeviceToDevice, stream);
        if (e != cudaSuccess) throw std::runtime_error(std::string("cudaMemcpyAsync: ") + cudaGetErrorString(e));
    }

    // the tensor as the C ABI takes it (one- and two-dimensional tensors; an undefined tensor has ndim 0)
    qmlp_tensor_t view() const
    {
        qmlp_tensor_t t{};
        if (!defined()) return t;
        if (ndim() > 2) throw std::runtime_error("only one- and two-dimensional tensors cross the C interface");
        t.data = data_;
        t.precision = precision_ == FLOAT ? QMLP_FLOAT : precision_ == HALF ? QMLP_HALF : QMLP_DOUBLE;
        t.ndim = ndim();
        for (int i = 0; i < ndim(); ++i) { t.sizes[i] = sizes_[i]; t.strides[i] = strides_[i]; }
        return t;
    }

private:
    template <typename T> void assertType() const
    {
        if (std::is_void<T>::value) return;
        if (precision_ == FLOAT && !std::is_same<float, T>::value) throw configuration_error("Illegal type, the tensor stores float data!");
        if (precision_ == HALF && !std::is_same<__half, T>::value) throw configuration_error("Illegal type, the tensor stores half data!");
        if (precision_ == DOUBLE && !std::is_same<double, T>::value) throw configuration_error("Illegal type, the tensor stores double data!");
    }

    void* data_ = nullptr;
    std::shared_ptr<void> owned_;
    Precision precision_ = FLOAT;
    std::vector<int32_t> sizes_, strides_;
};

} // namespace qmlp
