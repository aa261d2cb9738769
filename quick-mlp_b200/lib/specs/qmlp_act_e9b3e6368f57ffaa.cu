// stand-alone activation kernels for 'celu'
#include "standalone.cuh"
using namespace qmlp::kernel;
namespace {
namespace activations {
}
}
extern "C" int qmlp_spec_abi() { return QMLP_SPEC_ABI_VERSION; }
extern "C" int qmlp_spec_launch(int kernel, const void* args, cudaStream_t s, int* launches)
{ return ActivationLaunchers<BuiltinCelu>::launch(kernel, args, s, launches); }
