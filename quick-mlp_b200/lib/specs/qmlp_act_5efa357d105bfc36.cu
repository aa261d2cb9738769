// stand-alone activation kernels for 'sine'
#include "standalone.cuh"
using namespace qmlp::kernel;
namespace {
namespace activations {
}
}
extern "C" int qmlp_spec_abi() { return QMLP_SPEC_ABI_VERSION; }
extern "C" int qmlp_spec_launch(int kernel, const void* args, cudaStream_t s, int* launches)
{ return ActivationLaunchers<BuiltinSine>::launch(kernel, args, s, launches); }
