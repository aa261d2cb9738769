// stand-alone encoding kernels: {"id":"HashGrid","start_in":0,"n_in":3,"n_levels":8,"n_features_per_level":2,"log2_hashmap_size":10,"min_resolution":4,"max_resolution":512,"combination_mode":"concat","bounding_box_min":[0,0,0],"bounding_box_size":[1,1,1],"per_level_scale":2}
#include "standalone.cuh"
using namespace qmlp::kernel;
namespace {
struct EncSpec {
    static constexpr int NUM_ENCODINGS = 1;
    template <int E> struct Enc;
};
template <> struct EncSpec::Enc<0> : EncGrid<0, 3, 8, 2, true, 0, 0, false> {};
}
extern "C" int qmlp_spec_abi() { return QMLP_SPEC_ABI_VERSION; }
extern "C" int qmlp_spec_launch(int kernel, const void* args, cudaStream_t s, int* launches)
{ return EncodingLaunchers<EncSpec>::launch(kernel, args, s, launches); }
