// Plain structs shared by the host library and the per-spec kernel instantiations.
// They replace the reference's __constant__ HashGridConfig marshalling
// (src_cpp/include/qmlp/kernels/encoding_hashgrid_config.cuh:23-38, src_cpp/src/encoding_hashgrid.cpp:204-243):
// the level table travels as a __grid_constant__ kernel parameter instead of a cuMemcpyHtoDAsync per launch.
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace qmlp {
namespace kernel {

constexpr int MAX_GRID_LEVELS = 32;
constexpr int MAX_GRIDS = 4;
constexpr int MAX_GRID_DIMS = 6;

struct GridLevelP {
    unsigned int offset;       // element offset of the level inside the table (memoryOffset)
    int resolution;            // per-side resolution
    unsigned int hashGridSize; // rows if hashed (a power of two)
    int hashed;                // 1: hashed lookup, 0: dense lookup
};

struct GridP {
    const void* table; // fp32 (reference layout) or fp16 copy: [level0 rows*F | level1 ...]
    float* grad;       // fp32 gradient table, same layout (may be null)
    float boxMin[MAX_GRID_DIMS];
    float boxInvSize[MAX_GRID_DIMS];
    float boxSize[MAX_GRID_DIMS];
    float stepsize;    // line integration only: world-space step along the ray
    int tableIsHalf;
    int vecOk; // table and grad pointers are aligned for whole-row vector access
    unsigned long long tableCount; // elements of the table (and of its gradient): what QMLP_BOUNDS_CHECK builds check rows against
    int* status;                   // the library's status word (QMLP_BOUNDS_CHECK builds report through it), may be null
    GridLevelP levels[MAX_GRID_LEVELS];
};

// Bits of the library's device status word (qmlp_device_status). Bit 0 is set by a kernel that gave up on a bounded wait;
// the others only by instantiations compiled with QMLP_BOUNDS_CHECK, which test every table row, stash offset and plane
// offset against the size the host declared, skip an access that would leave it and report here instead of faulting.
constexpr int STATUS_WAIT_TIMEOUT = 1, STATUS_TABLE_ROW = 2, STATUS_STASH = 4, STATUS_PLANES = 8;
#ifdef QMLP_BOUNDS_CHECK
constexpr bool BOUNDS_CHECK = true;
#else
constexpr bool BOUNDS_CHECK = false;
#endif

// bits of LaunchArgs::flags for the backward kernel (AdjointMode of the reference,
// src_cpp/include/qmlp/fused_network.h:22-34)
constexpr int FLAG_GRAD_INPUT = 1;
constexpr int FLAG_GRAD_WEIGHTS = 2;
constexpr int FLAG_GRAD_ENCODINGS = 4;
// the backward kernel only writes the adjoint of the grid features to level-major planes (LaunchArgs::planes); the
// table gradients are scattered from there by KERNEL_SCATTER_PLANES. Only with FLAG_GRAD_ENCODINGS and without
// FLAG_GRAD_INPUT.
constexpr int FLAG_SPLIT_SCATTER = 8;

struct LaunchArgs {
    long long numel;
    const float* input;     long long inS0, inS1;
    float* output;          long long outS0, outS1;
    const float* adjOutput; long long aoS0, aoS1;
    float* adjInput;        long long aiS0, aiS1;
    const float* target;    long long tS0, tS1;   // fused L2 loss (training step)
    float lossScale;                               // 2 / (global points * channels)
    float* lossSum;                                // += sum (out-target)^2, may be null
    const __half* weights;                         // flat fp16 parameter vector
    float* gradWeights;                            // flat fp32 gradient vector
    __half* fwdTmp;                                // stash: encoded input + pre-activations per layer
    __half* adjTmp;                                // adjoint stash: delta per layer
    int flags;
    int numSMs;
    int numGrids;
    int forcePath;                                 // 0: best path for spec and batch, 1: mma.sync kernels only, 3: tcgen05 whenever instantiated
    int* status;                                   // device word set to 1 when a kernel gave up on a bounded wait
    __half* planes;                                // encoded features (or their adjoints) of a chunk of points, one plane per grid level
    long long planeStride;                         // points per plane (capacity of the chunk buffer)
    long long fwdTmpHalfs, adjTmpHalfs, planeHalfs; // sizes of the three scratch buffers in halfs (QMLP_BOUNDS_CHECK builds; 0: unknown)
    // spatially binned training step (kernels/sorted_scatter.cuh): KERNEL_SORT_POINTS copies the points (and targets)
    // into Morton-bin order; the kernels after it read the sorted copies through `input` / `target`
    unsigned int* binCounts;                       // points per bin (sort_bin_count() entries), zeroed by the launcher
    unsigned int* binStart;                        // first sorted point of every bin, sort_bin_count() + 1 entries
    unsigned int* binCursor;                       // running insert position per bin
    float* sortedInput;                            // (numel, NUM_INPUTS) row-major
    float* sortedTarget;                           // (numel, NUM_OUTPUTS) row-major, may be null
    int scatterLevelBegin, scatterLevelEnd;        // KERNEL_SCATTER_PLANES: grid levels (counted over all grids) to scatter; 0, 0 = all
    int runAggregation;                            // 0: every point of every level scatters straight to the gradient table
    GridP grids[MAX_GRIDS];
};

// Bins of the point sort: a regular grid of 2^sort_bin_bits(D) cells per dimension over the bounding box of the first
// grid encoding, numbered in Morton order (bit b of dimension d at bit b * D + d of the key).
__host__ __device__ constexpr int sort_bin_bits(int dims)
{
    return dims <= 1 ? 16 : dims == 2 ? 9 : dims == 3 ? 6 : dims == 4 ? 4 : 3;
}
__host__ __device__ constexpr int sort_bin_count(int dims) { return 1 << (sort_bin_bits(dims) * dims); }

// kernels a network instantiation exports through qmlp_spec_launch
enum KernelId {
    KERNEL_INFERENCE = 0,
    KERNEL_FORWARD = 1,       // forward with stash
    KERNEL_FORWARD_LOSS = 2,  // forward with stash, writes dLoss/dOut of the L2 loss instead of the output
    KERNEL_BACKWARD = 3,      // flags select the variant
    KERNEL_WGRAD = 4,
    KERNEL_ENCODING_FORWARD = 5,
    KERNEL_ENCODING_ADJOINT = 6,
    KERNEL_ACTIVATION_FORWARD = 7,
    KERNEL_ACTIVATION_ADJOINT = 8,
    KERNEL_ENCODE_PLANES = 9,      // encodings of a chunk of points -> level-major feature planes
    KERNEL_INFERENCE_PLANES = 10,  // layer chain reading the feature planes instead of running the encodings
    KERNEL_SCATTER_PLANES = 11,    // adjoint feature planes -> grid table gradients, one grid level at a time
    KERNEL_FORWARD_LOSS_PLANES = 12, // KERNEL_FORWARD_LOSS with layer 0 fed from the planes of KERNEL_ENCODE_PLANES
    KERNEL_SORT_POINTS = 13,         // points (and targets) -> Morton-bin order: count, scan, reorder
    KERNEL_SCATTER_SORTED = 15       // KERNEL_SCATTER_PLANES for sorted points: coarse levels summed in shared memory first
};

// arguments of the stand-alone activation kernels
struct ActivationArgs {
    long long rows, cols;
    const __half* input;     long long inS0, inS1;
    const __half* adjOutput; long long aoS0, aoS1;
    __half* output;          long long outS0, outS1; // forward: z; adjoint: adjx
};

} // namespace kernel
} // namespace qmlp

// entry points every instantiation exports
extern "C" {
typedef int (*qmlp_spec_launch_fn)(int kernel, const void* args, cudaStream_t stream, int* launches);
typedef int (*qmlp_spec_abi_fn)(void);
}
#define QMLP_SPEC_ABI_VERSION 9
