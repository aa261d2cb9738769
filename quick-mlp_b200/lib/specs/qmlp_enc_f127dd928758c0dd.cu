// stand-alone encoding kernels: {"id":"Identity","start_in":1,"n_in":5}
#include "standalone.cuh"
using namespace qmlp::kernel;
namespace {
struct EncSpec {
    static constexpr int NUM_ENCODINGS = 1;
    template <int E> struct Enc;
};
template <> struct EncSpec::Enc<0> : EncIdentity<1, 5, 0> {};
}
extern "C" int qmlp_spec_abi() { return QMLP_SPEC_ABI_VERSION; }
extern "C" int qmlp_spec_launch(int kernel, const void* args, cudaStream_t s, int* launches)
{ return EncodingLaunchers<EncSpec>::launch(kernel, args, s, launches); }
