// fused-network instantiation; layers: 16->64+b:relu 64->64+b:celu 64->64+b:sine 64->64+b:relu 64->16+b:identity
#include "standalone.cuh"
using namespace qmlp::kernel;
namespace {
namespace activations {
}
struct Spec {
    static constexpr int NUM_INPUTS = 3, NUM_OUTPUTS = 1, NUM_LAYERS = 5, ENC_CHANNELS = 3, NUM_ENCODINGS = 1;
    static constexpr int WARPS = 8, MIN_BLOCKS = 2;
    static constexpr int CIN[5] = {16, 64, 64, 64, 64};
    static constexpr int COUT[5] = {64, 64, 64, 64, 16};
    static constexpr int WOFF[5] = {0, 1024, 5120, 9216, 13312};
    static constexpr int BOFF[5] = {14336, 14400, 14464, 14528, 14592};
    template <int L> struct Act;
    template <int E> struct Enc;
};
template <> struct Spec::Act<0> : BuiltinRelu {};
template <> struct Spec::Act<1> : BuiltinCelu {};
template <> struct Spec::Act<2> : BuiltinSine {};
template <> struct Spec::Act<3> : BuiltinRelu {};
template <> struct Spec::Act<4> : BuiltinIdentity {};
template <> struct Spec::Enc<0> : EncIdentity<0, 3, 0> {};
}
extern "C" int qmlp_spec_abi() { return QMLP_SPEC_ABI_VERSION; }
extern "C" int qmlp_spec_launch(int kernel, const void* args, cudaStream_t s, int* launches)
{ return NetworkLaunchers<Spec>::launch(kernel, args, s, launches); }
