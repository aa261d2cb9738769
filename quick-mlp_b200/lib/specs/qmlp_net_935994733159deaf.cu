// fused-network instantiation; layers: 16->32:celu 32->48:identity 48->16:celu
#include "standalone.cuh"
using namespace qmlp::kernel;
namespace {
namespace activations {
}
struct Spec {
    static constexpr int NUM_INPUTS = 16, NUM_OUTPUTS = 16, NUM_LAYERS = 3, ENC_CHANNELS = 16, NUM_ENCODINGS = 1;
    static constexpr int WARPS = 8, MIN_BLOCKS = 2;
    static constexpr int CIN[3] = {16, 32, 48};
    static constexpr int COUT[3] = {32, 48, 16};
    static constexpr int WOFF[3] = {0, 512, 2048};
    static constexpr int BOFF[3] = {-1, -1, -1};
    template <int L> struct Act;
    template <int E> struct Enc;
};
template <> struct Spec::Act<0> : BuiltinCelu {};
template <> struct Spec::Act<1> : BuiltinIdentity {};
template <> struct Spec::Act<2> : BuiltinCelu {};
template <> struct Spec::Enc<0> : EncIdentity<0, 16, 0> {};
}
extern "C" int qmlp_spec_abi() { return QMLP_SPEC_ABI_VERSION; }
extern "C" int qmlp_spec_launch(int kernel, const void* args, cudaStream_t s, int* launches)
{ return NetworkLaunchers<Spec>::launch(kernel, args, s, launches); }
