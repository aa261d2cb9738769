// fused-network instantiation; layers: 64->128+b:relu 128->128+b:relu 128->128+b:relu 128->16+b:identity
#include "standalone.cuh"
using namespace qmlp::kernel;
namespace {
namespace activations {
}
struct Spec {
    static constexpr int NUM_INPUTS = 4, NUM_OUTPUTS = 4, NUM_LAYERS = 4, ENC_CHANNELS = 64, NUM_ENCODINGS = 1;
    static constexpr int WARPS = 8, MIN_BLOCKS = 1;
    static constexpr int CIN[4] = {64, 128, 128, 128};
    static constexpr int COUT[4] = {128, 128, 128, 16};
    static constexpr int WOFF[4] = {0, 8192, 24576, 40960};
    static constexpr int BOFF[4] = {43008, 43136, 43264, 43392};
    template <int L> struct Act;
    template <int E> struct Enc;
};
template <> struct Spec::Act<0> : BuiltinRelu {};
template <> struct Spec::Act<1> : BuiltinRelu {};
template <> struct Spec::Act<2> : BuiltinRelu {};
template <> struct Spec::Act<3> : BuiltinIdentity {};
template <> struct Spec::Enc<0> : EncGrid<0, 4, 16, 4, true, 0, 0, true> {};
}
extern "C" int qmlp_spec_abi() { return QMLP_SPEC_ABI_VERSION; }
extern "C" int qmlp_spec_launch(int kernel, const void* args, cudaStream_t s, int* launches)
{ return NetworkLaunchers<Spec>::launch(kernel, args, s, launches); }
