// stand-alone activation kernels for 'leaky'
#include "standalone.cuh"
using namespace qmlp::kernel;
namespace {
namespace activations {
struct leaky {
    static __device__ __forceinline__ half forward(half x) { half z; z = __hgt(x, hZERO()) ? x : __hmul(x, __float2half(0.125f)) ; return z; }
    static __device__ __forceinline__ half adjoint(half x, half adjz) { half adjx; adjx = __hgt(x, hZERO()) ? adjz : __hmul(adjz, __float2half(0.125f)) ; return adjx; }
};
}
}
extern "C" int qmlp_spec_abi() { return QMLP_SPEC_ABI_VERSION; }
extern "C" int qmlp_spec_launch(int kernel, const void* args, cudaStream_t s, int* launches)
{ return ActivationLaunchers<ScalarActivation<activations::leaky>>::launch(kernel, args, s, launches); }
