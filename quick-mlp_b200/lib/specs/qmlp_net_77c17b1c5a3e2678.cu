// fused-network instantiation; layers: 16->32+b:sine 32->32:relu 32->16+b:identity
#include "standalone.cuh"
using namespace qmlp::kernel;
namespace {
namespace activations {
}
struct Spec {
    static constexpr int NUM_INPUTS = 5, NUM_OUTPUTS = 7, NUM_LAYERS = 3, ENC_CHANNELS = 5, NUM_ENCODINGS = 1;
    static constexpr int WARPS = 8, MIN_BLOCKS = 2;
    static constexpr int CIN[3] = {16, 32, 32};
    static constexpr int COUT[3] = {32, 32, 16};
    static constexpr int WOFF[3] = {0, 512, 1536};
    static constexpr int BOFF[3] = {2048, -1, 2080};
    template <int L> struct Act;
    template <int E> struct Enc;
};
template <> struct Spec::Act<0> : BuiltinSine {};
template <> struct Spec::Act<1> : BuiltinRelu {};
template <> struct Spec::Act<2> : BuiltinIdentity {};
template <> struct Spec::Enc<0> : EncIdentity<0, 5, 0> {};
}
extern "C" int qmlp_spec_abi() { return QMLP_SPEC_ABI_VERSION; }
extern "C" int qmlp_spec_launch(int kernel, const void* args, cudaStream_t s, int* launches)
{ return NetworkLaunchers<Spec>::launch(kernel, args, s, launches); }
