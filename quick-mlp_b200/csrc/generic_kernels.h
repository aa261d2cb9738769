// Launchers of the spec-independent kernels (Adam, master -> half refresh).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace qmlp {
namespace kernel {

// `count` must be a multiple of 4 and all pointers 16-byte aligned (8-byte for halfCopy).
cudaError_t launchAdam(float* master, float* grad, float* m, float* v, uint16_t* halfCopy, long long count,
                       float gradScale, float beta1, float beta2, float stepSize, float invSqrtBc2, float eps,
                       int numSMs, cudaStream_t stream);
// Address, on the current device, of the library's kernel status word (a __device__ variable).
cudaError_t statusWordAddress(int** out);
cudaError_t launchRefreshHalf(const float* master, uint16_t* halfCopy, long long count, int numSMs, cudaStream_t stream);

} // namespace kernel
} // namespace qmlp
