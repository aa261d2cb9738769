// Spec-independent kernels of the fused training step: Adam over the fused parameter buffer and the
// master -> half refresh. The reference has no counterpart: there the optimiser is torch.optim.Adam in user code
// (tests_py/qmlp_tests/test_network_image.py:43,51-53); the update rule below is the one torch.optim.Adam applies
// (no amsgrad, no weight decay).
#include "generic_kernels.h"

#include <cuda_fp16.h>

namespace qmlp {
namespace kernel {

// One pass: g *= gradScale; m, v update; master -= stepSize * m / (sqrt(v) * invSqrtBc2 + eps); half copy; g = 0.
// HBM traffic per element: 16 B read (p, g, m, v) + 14 B written (p, m, v, half, and the zeroed g).
__global__ void __launch_bounds__(256) adam_kernel(float4* __restrict__ master, float4* __restrict__ grad,
                                                   float4* __restrict__ m, float4* __restrict__ v,
                                                   uint2* __restrict__ halfCopy, long long count4, float gradScale,
                                                   float beta1, float beta2, float stepSize, float invSqrtBc2, float eps)
{
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < count4;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
        float4 g = grad[i];
        float4 p = master[i], mm = m[i], vv = v[i];
        float* gp = reinterpret_cast<float*>(&g);
        float* pp = reinterpret_cast<float*>(&p);
        float* mp = reinterpret_cast<float*>(&mm);
        float* vp = reinterpret_cast<float*>(&vv);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const float gk = gp[k] * gradScale;
            mp[k] = beta1 * mp[k] + (1.f - beta1) * gk;
            vp[k] = beta2 * vp[k] + (1.f - beta2) * gk * gk;
            const float denom = sqrtf(vp[k]) * invSqrtBc2 + eps;
            pp[k] -= stepSize * (mp[k] / denom);
        }
        master[i] = p;
        m[i] = mm;
        v[i] = vv;
        grad[i] = make_float4(0.f, 0.f, 0.f, 0.f);
        __half2 h0 = __floats2half2_rn(pp[0], pp[1]), h1 = __floats2half2_rn(pp[2], pp[3]);
        uint2 u;
        u.x = *reinterpret_cast<unsigned int*>(&h0);
        u.y = *reinterpret_cast<unsigned int*>(&h1);
        halfCopy[i] = u;
    }
}

__global__ void __launch_bounds__(256) refresh_half_kernel(const float4* __restrict__ master, uint2* __restrict__ halfCopy,
                                                           long long count4)
{
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < count4;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
        const float4 p = master[i];
        __half2 h0 = __floats2half2_rn(p.x, p.y), h1 = __floats2half2_rn(p.z, p.w);
        uint2 u;
        u.x = *reinterpret_cast<unsigned int*>(&h0);
        u.y = *reinterpret_cast<unsigned int*>(&h1);
        halfCopy[i] = u;
    }
}

// set to 1 by a kernel that gave up on a bounded on-chip wait; one copy per device context that loads the library
static __device__ int g_statusWord;

cudaError_t statusWordAddress(int** out) { return cudaGetSymbolAddress(reinterpret_cast<void**>(out), g_statusWord); }

static unsigned gridFor(long long work, int numSMs)
{
    long long blocks = (work + 255) / 256;
    const long long cap = static_cast<long long>(numSMs) * 8;
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    return static_cast<unsigned>(blocks);
}

cudaError_t launchAdam(float* master, float* grad, float* m, float* v, uint16_t* halfCopy, long long count,
                       float gradScale, float beta1, float beta2, float stepSize, float invSqrtBc2, float eps,
                       int numSMs, cudaStream_t stream)
{
    const long long count4 = count / 4;
    adam_kernel<<<gridFor(count4, numSMs), 256, 0, stream>>>(
        reinterpret_cast<float4*>(master), reinterpret_cast<float4*>(grad), reinterpret_cast<float4*>(m),
        reinterpret_cast<float4*>(v), reinterpret_cast<uint2*>(halfCopy), count4, gradScale, beta1, beta2, stepSize,
        invSqrtBc2, eps);
    return cudaGetLastError();
}

cudaError_t launchRefreshHalf(const float* master, uint16_t* halfCopy, long long count, int numSMs, cudaStream_t stream)
{
    const long long count4 = count / 4;
    refresh_half_kernel<<<gridFor(count4, numSMs), 256, 0, stream>>>(reinterpret_cast<const float4*>(master),
                                                                     reinterpret_cast<uint2*>(halfCopy), count4);
    return cudaGetLastError();
}

} // namespace kernel
} // namespace qmlp
