// stand-alone encoding kernels: {"id":"HashGrid","start_in":2,"n_in":3,"n_levels":4,"n_features_per_level":3,"log2_hashmap_size":9,"min_resolution":8,"max_resolution":128,"combination_mode":"add","bounding_box_min":[-2,-2,-2],"bounding_box_size":[4,4,4]}
#include "standalone.cuh"
using namespace qmlp::kernel;
namespace {
struct EncSpec {
    static constexpr int NUM_ENCODINGS = 1;
    template <int E> struct Enc;
};
template <> struct EncSpec::Enc<0> : EncGrid<2, 3, 4, 3, false, 0, 0, false> {};
}
extern "C" int qmlp_spec_abi() { return QMLP_SPEC_ABI_VERSION; }
extern "C" int qmlp_spec_launch(int kernel, const void* args, cudaStream_t s, int* launches)
{ return EncodingLaunchers<EncSpec>::launch(kernel, args, s, launches); }
