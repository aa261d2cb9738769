// fused-network instantiation; layers: 48->128+b:sine 128->64+b:celu 64->16+b:relu 16->16+b:identity
#include "standalone.cuh"
using namespace qmlp::kernel;
namespace {
namespace activations {
}
struct Spec {
    static constexpr int NUM_INPUTS = 3, NUM_OUTPUTS = 4, NUM_LAYERS = 4, ENC_CHANNELS = 36, NUM_ENCODINGS = 2;
    static constexpr int WARPS = 8, MIN_BLOCKS = 1;
    static constexpr int CIN[4] = {48, 128, 64, 16};
    static constexpr int COUT[4] = {128, 64, 16, 16};
    static constexpr int WOFF[4] = {0, 6144, 14336, 15360};
    static constexpr int BOFF[4] = {15616, 15744, 15808, 15824};
    template <int L> struct Act;
    template <int E> struct Enc;
};
template <> struct Spec::Act<0> : BuiltinSine {};
template <> struct Spec::Act<1> : BuiltinCelu {};
template <> struct Spec::Act<2> : BuiltinRelu {};
template <> struct Spec::Act<3> : BuiltinIdentity {};
template <> struct Spec::Enc<0> : EncGrid<0, 3, 1, 4, true, 0, 0, false> {};
template <> struct Spec::Enc<1> : EncGrid<0, 3, 8, 4, true, 4, 1, false> {};
}
extern "C" int qmlp_spec_abi() { return QMLP_SPEC_ABI_VERSION; }
extern "C" int qmlp_spec_launch(int kernel, const void* args, cudaStream_t s, int* launches)
{ return NetworkLaunchers<Spec>::launch(kernel, args, s, launches); }
