// stand-alone encoding kernels: {"id":"HashGrid","start_in":0,"n_in":2,"n_levels":1,"n_features_per_level":4,"log2_hashmap_size":-1,"min_resolution":2,"max_resolution":16,"combination_mode":"add","bounding_box_min":[-1,-1],"bounding_box_size":[2,2]}
#include "standalone.cuh"
using namespace qmlp::kernel;
namespace {
struct EncSpec {
    static constexpr int NUM_ENCODINGS = 1;
    template <int E> struct Enc;
};
template <> struct EncSpec::Enc<0> : EncGrid<0, 2, 1, 4, false, 0, 0, false> {};
}
extern "C" int qmlp_spec_abi() { return QMLP_SPEC_ABI_VERSION; }
extern "C" int qmlp_spec_launch(int kernel, const void* args, cudaStream_t s, int* launches)
{ return EncodingLaunchers<EncSpec>::launch(kernel, args, s, launches); }
