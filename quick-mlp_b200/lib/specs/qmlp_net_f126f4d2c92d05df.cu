// fused-network instantiation; layers: 32->64+b:relu 64->64+b:relu 64->16+b:identity
#include "standalone.cuh"
using namespace qmlp::kernel;
namespace {
namespace activations {
}
struct Spec {
    static constexpr int NUM_INPUTS = 3, NUM_OUTPUTS = 1, NUM_LAYERS = 3, ENC_CHANNELS = 32, NUM_ENCODINGS = 1;
    static constexpr int WARPS = 8, MIN_BLOCKS = 2;
    static constexpr int CIN[3] = {32, 64, 64};
    static constexpr int COUT[3] = {64, 64, 16};
    static constexpr int WOFF[3] = {0, 2048, 6144};
    static constexpr int BOFF[3] = {7168, 7232, 7296};
    template <int L> struct Act;
    template <int E> struct Enc;
};
template <> struct Spec::Act<0> : BuiltinRelu {};
template <> struct Spec::Act<1> : BuiltinRelu {};
template <> struct Spec::Act<2> : BuiltinIdentity {};
template <> struct Spec::Enc<0> : EncGrid<0, 3, 16, 2, true, 0, 0, false> {};
}
extern "C" int qmlp_spec_abi() { return QMLP_SPEC_ABI_VERSION; }
extern "C" int qmlp_spec_launch(int kernel, const void* args, cudaStream_t s, int* launches)
{ return NetworkLaunchers<Spec>::launch(kernel, args, s, launches); }
