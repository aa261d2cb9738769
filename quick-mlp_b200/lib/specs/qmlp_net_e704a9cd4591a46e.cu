// fused-network instantiation; layers: 16->32+b:leaky 32->32+b:sine 32->16+b:leaky
#include "standalone.cuh"
using namespace qmlp::kernel;
namespace {
namespace activations {
struct leaky {
    static __device__ __forceinline__ half forward(half x) { half z; z = __hgt(x, hZERO()) ? x : __hmul(x, __float2half(0.125f)) ; return z; }
    static __device__ __forceinline__ half adjoint(half x, half adjz) { half adjx; adjx = __hgt(x, hZERO()) ? adjz : __hmul(adjz, __float2half(0.125f)) ; return adjx; }
};
}
struct Spec {
    static constexpr int NUM_INPUTS = 4, NUM_OUTPUTS = 2, NUM_LAYERS = 3, ENC_CHANNELS = 4, NUM_ENCODINGS = 1;
    static constexpr int WARPS = 8, MIN_BLOCKS = 2;
    static constexpr int CIN[3] = {16, 32, 32};
    static constexpr int COUT[3] = {32, 32, 16};
    static constexpr int WOFF[3] = {0, 512, 1536};
    static constexpr int BOFF[3] = {2048, 2080, 2112};
    template <int L> struct Act;
    template <int E> struct Enc;
};
template <> struct Spec::Act<0> : ScalarActivation<activations::leaky> {};
template <> struct Spec::Act<1> : BuiltinSine {};
template <> struct Spec::Act<2> : ScalarActivation<activations::leaky> {};
template <> struct Spec::Enc<0> : EncIdentity<0, 4, 0> {};
}
extern "C" int qmlp_spec_abi() { return QMLP_SPEC_ABI_VERSION; }
extern "C" int qmlp_spec_launch(int kernel, const void* args, cudaStream_t s, int* launches)
{ return NetworkLaunchers<Spec>::launch(kernel, args, s, launches); }
