// Stand-alone (non-fused) encoding and activation kernels.
// They replace EncodingForwardKernel / EncodingAdjointKernel (src_cpp/include/qmlp/kernels/encoding_kernels.cuh:26-62,
// launched by src_cpp/src/iencoding.cpp:12-196) and ActivationForwardKernel / ActivationAdjointKernel
// (src_cpp/include/qmlp/kernels/activation_kernels.cuh:28-62, launched by src_cpp/src/activation.cpp:64-150).
#pragma once
#include "fused_network.cuh"
#include "fused_forward_tc.cuh"

namespace qmlp {
namespace kernel {

struct FloatRowWriter {
    float* row; long long s1;
    __device__ __forceinline__ void operator()(int c, float v) const { row[c * s1] = v; }
};
struct FloatRowReader {
    const float* row; long long s1;
    __device__ __forceinline__ float operator()(int c) const { return __ldg(row + c * s1); }
};

// EncSpec: NUM_ENCODINGS == 1 and Enc<0>
template <class EncSpec>
__global__ void __launch_bounds__(256) encoding_forward_kernel(const __grid_constant__ LaunchArgs p)
{
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < p.numel;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
        RowReader in{p.input + i * p.inS0, p.inS1};
        encode_point<EncSpec, 0>(p, in, FloatRowWriter{p.output + i * p.outS0, p.outS1});
    }
}

template <class EncSpec, bool INPUT_GRAD, bool PARAM_GRAD>
__global__ void __launch_bounds__(256) encoding_adjoint_kernel(const __grid_constant__ LaunchArgs p)
{
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < p.numel;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
        RowReader in{p.input + i * p.inS0, p.inS1};
        float* adjInRow = INPUT_GRAD ? p.adjInput + i * p.aiS0 : nullptr;
        encode_adjoint_point<EncSpec, 0, INPUT_GRAD, PARAM_GRAD>(
            p, in, FloatRowReader{p.adjOutput + i * p.aoS0, p.aoS1}, adjInRow, p.aiS1);
    }
}

template <class EncSpec>
struct EncodingLaunchers {
    static int launch(int kernel, const void* args, cudaStream_t s, int* launches)
    {
        const LaunchArgs& a = *static_cast<const LaunchArgs*>(args);
        long long blocks = (a.numel + 255) / 256;
        const long long cap = static_cast<long long>(a.numSMs) * 8;
        if (blocks > cap) blocks = cap;
        if (blocks < 1) blocks = 1;
        const unsigned g = static_cast<unsigned>(blocks);
        if (kernel == KERNEL_ENCODING_FORWARD) {
            encoding_forward_kernel<EncSpec><<<g, 256, 0, s>>>(a);
        } else if (kernel == KERNEL_ENCODING_ADJOINT) {
            const bool ig = (a.flags & 1) != 0, pg = (a.flags & 2) != 0;
            if (ig && pg) encoding_adjoint_kernel<EncSpec, true, true><<<g, 256, 0, s>>>(a);
            else if (ig) encoding_adjoint_kernel<EncSpec, true, false><<<g, 256, 0, s>>>(a);
            else if (pg) encoding_adjoint_kernel<EncSpec, false, true><<<g, 256, 0, s>>>(a);
            else { if (launches) *launches = 0; return 0; }
        } else {
            if (launches) *launches = 0;
            return static_cast<int>(cudaErrorInvalidValue);
        }
        cudaError_t e = cudaGetLastError();
        if (launches) *launches = e == cudaSuccess ? 1 : 0;
        return static_cast<int>(e);
    }
};

// element-wise half activation over an (N, C) tensor with arbitrary strides
template <class Act, bool ADJOINT>
__global__ void __launch_bounds__(256) activation_kernel(const __grid_constant__ ActivationArgs p)
{
    const long long total = p.rows * p.cols;
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
        const long long r = i / p.cols, c = i % p.cols;
        const half x = p.input[r * p.inS0 + c * p.inS1];
        if constexpr (ADJOINT) {
            const half g = p.adjOutput[r * p.aoS0 + c * p.aoS1];
            p.output[r * p.outS0 + c * p.outS1] = Act::adjoint(x, g);
        } else {
            p.output[r * p.outS0 + c * p.outS1] = Act::forward(x);
        }
    }
}

// contiguous fast path: half2 vectorised
template <class Act, bool ADJOINT>
__global__ void __launch_bounds__(256) activation_kernel_vec(const __grid_constant__ ActivationArgs p)
{
    const long long total2 = p.rows * p.cols / 2;
    const __half2* in = reinterpret_cast<const __half2*>(p.input);
    const __half2* go = reinterpret_cast<const __half2*>(p.adjOutput);
    __half2* out = reinterpret_cast<__half2*>(p.output);
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total2;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
        if constexpr (ADJOINT) out[i] = Act::adjoint2(in[i], go[i]);
        else out[i] = Act::forward2(in[i]);
    }
}

template <class Act>
struct ActivationLaunchers {
    static int launch(int kernel, const void* args, cudaStream_t s, int* launches)
    {
        const ActivationArgs& a = *static_cast<const ActivationArgs*>(args);
        const long long total = a.rows * a.cols;
        if (total == 0) { if (launches) *launches = 0; return 0; }
        const bool adj = kernel == KERNEL_ACTIVATION_ADJOINT;
        auto contiguous = [&](long long s0, long long s1) { return s1 == 1 && s0 == a.cols; };
        auto aligned4 = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 3) == 0; };
        bool vec = (total % 2 == 0) && contiguous(a.inS0, a.inS1) && contiguous(a.outS0, a.outS1) && aligned4(a.input) && aligned4(a.output);
        if (adj) vec = vec && contiguous(a.aoS0, a.aoS1) && aligned4(a.adjOutput);
        const long long work = vec ? total / 2 : total;
        long long blocks = (work + 255) / 256;
        if (blocks > 148 * 16) blocks = 148 * 16;
        const unsigned g = static_cast<unsigned>(blocks);
        if (kernel == KERNEL_ACTIVATION_FORWARD) {
            if (vec) activation_kernel_vec<Act, false><<<g, 256, 0, s>>>(a);
            else activation_kernel<Act, false><<<g, 256, 0, s>>>(a);
        } else if (adj) {
            if (vec) activation_kernel_vec<Act, true><<<g, 256, 0, s>>>(a);
            else activation_kernel<Act, true><<<g, 256, 0, s>>>(a);
        } else {
            if (launches) *launches = 0;
            return static_cast<int>(cudaErrorInvalidValue);
        }
        cudaError_t e = cudaGetLastError();
        if (launches) *launches = e == cudaSuccess ? 1 : 0;
        return static_cast<int>(e);
    }
};

} // namespace kernel
} // namespace qmlp
