// Fused network kernels: encodings -> fully-connected layer chain, forward and adjoint.
//
// They replace the reference's NetworkKernelInferenceAndForward (src_cpp/include/qmlp/kernels/network_forward.cuh:34-114),
// NetworkKernelBackward (kernels/network_backward.cuh:33-114) and Layer<>::inference/adjoint (kernels/layer.cuh:101-265).
//
// Design (not the reference's): a persistent grid; every CTA stages all weight matrices and biases of the network
// in shared memory once; every warp then works alone on tiles of 32 points. The activations of a tile never leave
// registers between layers: the fp32 accumulator fragment of one m16n8k16 MMA, rounded to half2 and passed through
// the activation, is exactly the A-operand fragment of the next layer. Weights are read from shared memory with
// ldmatrix (forward) and ldmatrix.trans (adjoint, W^T) from one row-major copy. Accumulation is fp32 (the reference
// accumulates in half).
//
// A `Spec` type, generated per network, supplies the compile-time geometry:
//   NUM_INPUTS, NUM_OUTPUTS, NUM_LAYERS, ENC_CHANNELS, NUM_ENCODINGS, WARPS, MIN_BLOCKS
//   CIN[l], COUT[l] (padded to 16), WOFF[l], BOFF[l] (-1: no bias)   -- offsets into the flat parameter vector
//   template<int L> struct Act  : activation functor of layer L
//   template<int E> struct Enc  : EncIdentity<...> or EncGrid<...>
#pragma once
#include <atomic>

#include "launch_args.h"
#include "mma.cuh"
#include "activations.cuh"
#include "grid.cuh"

namespace qmlp {
namespace kernel {

constexpr int TILE_POINTS = 32; // points per warp tile = 2 MMA row tiles
constexpr int MT = 2;

// ---- encoding descriptors ------------------------------------------------------------------------------------
template <int START_, int N_, int OUT_OFF_>
struct EncIdentity {
    static constexpr bool IS_GRID = false, IS_LINE = false;
    static constexpr int START = START_, N = N_, OUT_OFF = OUT_OFF_, NUM_OUT = N_;
};
template <int START_, int D_, int L_, int F_, bool CONCAT_, int OUT_OFF_, int SLOT_, bool HALF_TABLE_>
struct EncGrid {
    static constexpr bool IS_GRID = true, IS_LINE = false;
    static constexpr int START = START_, D = D_, L = L_, F = F_, OUT_OFF = OUT_OFF_, SLOT = SLOT_;
    static constexpr bool CONCAT = CONCAT_, HALF_TABLE = HALF_TABLE_;
    static constexpr int NUM_OUT = CONCAT_ ? L_ * F_ : F_;
};

// Line integration over a grid (src_cpp/include/qmlp/kernels/encoding_line_integration.cuh:51-166): the input holds a
// ray start and a ray direction (2 * D channels from START); the grid is sampled every GridP::stepsize along the part of
// the ray inside the grid's bounding box and the samples are summed (AVERAGE: divided by the number of steps).
template <int START_, int D_, int L_, int F_, bool CONCAT_, int OUT_OFF_, int SLOT_, bool HALF_TABLE_, bool AVERAGE_>
struct EncLine {
    static constexpr bool IS_GRID = false, IS_LINE = true;
    static constexpr int START = START_, D = D_, L = L_, F = F_, OUT_OFF = OUT_OFF_, SLOT = SLOT_;
    static constexpr bool CONCAT = CONCAT_, HALF_TABLE = HALF_TABLE_, AVERAGE = AVERAGE_;
    static constexpr int NUM_OUT = CONCAT_ ? L_ * F_ : F_;
    static_assert(D_ == 3, "the ray / bounding-box intersection exists for three dimensions only");
};

// ---- shared memory layout ------------------------------------------------------------------------------------
// weights of layer l: [COUT][CIN + 8] halfs (row padded by 16 bytes: conflict-free ldmatrix), then the biases (half),
// then one [32][CIN0 + 8] half tile per warp.
template <class Spec>
struct SmemLayout {
    static constexpr int NL = Spec::NUM_LAYERS;
    __host__ __device__ static constexpr int wStride(int l) { return Spec::CIN[l] + 8; }
    __host__ __device__ static constexpr int wOffsetHalfs(int l)
    {
        int o = 0;
        for (int i = 0; i < l; ++i) o += Spec::COUT[i] * (Spec::CIN[i] + 8);
        return o;
    }
    __host__ __device__ static constexpr int weightHalfs() { return wOffsetHalfs(NL); }
    __host__ __device__ static constexpr int biasOffset(int l)
    {
        int o = 0;
        for (int i = 0; i < l; ++i) o += Spec::COUT[i];
        return o;
    }
    __host__ __device__ static constexpr int biasHalfs() { return biasOffset(NL); }
    __host__ __device__ static constexpr int biasStartBytes() { return ((weightHalfs() * 2 + 15) / 16) * 16; }
    __host__ __device__ static constexpr int tileStride() { return Spec::CIN[0] + 8; }
    __host__ __device__ static constexpr int tileStartBytes() { return ((biasStartBytes() + biasHalfs() * 2 + 15) / 16) * 16; }
    __host__ __device__ static constexpr int tileBytesPerWarp() { return TILE_POINTS * tileStride() * 2; }
    __host__ __device__ static constexpr int totalBytes() { return tileStartBytes() + Spec::WARPS * tileBytesPerWarp(); }
    // prefix sums of the stash (in halfs per point)
    __host__ __device__ static constexpr int preOffset(int l)
    { // encoded input first, then the pre-activations of every layer
        int o = Spec::CIN[0];
        for (int i = 0; i < l; ++i) o += Spec::COUT[i];
        return o;
    }
    __host__ __device__ static constexpr int deltaOffset(int l)
    {
        int o = 0;
        for (int i = 0; i < l; ++i) o += Spec::COUT[i];
        return o;
    }
};

// Layout of a pre-activation or delta matrix (N32 points x C channels, halfs) in the stash: tiles of 32 points, each
// tile cut into blocks of 8 points x 8 channels that are stored contiguously (128 bytes, point-major), block (cb, rb) of
// a tile at ((cb * 4 + rb) * 64) halfs. An m16n8k16 accumulator / A fragment register of a warp (lane = 4 * r + q holds
// row r, columns 2 q and 2 q + 1 of an 8 x 8 block) then covers exactly one block, so the 4-byte accesses of a warp
// are one contiguous 128-byte line: four sector requests instead of the eight half-filled ones a row-major matrix
// costs. The forward and backward kernels are bound by the rate of such requests (one per clock and SM), and the stash
// accounted for a third of them. A row of 8 channels is still one 16-byte piece, which is what wgrad_kernel copies.
__host__ __device__ __forceinline__ long long stash_block(long long tileRow0, int channels, int rb, int cb)
{
    return tileRow0 * channels + (cb * 4 + rb) * 64;
}

// QMLP_BOUNDS_CHECK builds: does [offset, offset + count) lie inside a scratch buffer of `capacity` halfs (0: the host gave
// no size)? If not, the status word gets `bit` and the caller skips the access. Compiles to `true` in regular builds.
__device__ __forceinline__ bool scratch_ok(const LaunchArgs& p, long long offset, int count, long long capacity, int bit)
{
    if constexpr (BOUNDS_CHECK) {
        if (capacity > 0 && (offset < 0 || offset + count > capacity)) {
            if (p.status != nullptr) atomicOr(p.status, bit);
            return false;
        }
    }
    (void)p; (void)offset; (void)count; (void)capacity; (void)bit;
    return true;
}

// CTAs per SM the forward and backward kernels are compiled for: two (a 128-register budget per thread, which costs
// the 128-wide networks a few dozen bytes of spills but doubles the warps that hide gather and stash latency) whenever
// two copies of the shared-memory plan fit on an SM, else one.
template <class Spec>
__host__ __device__ constexpr int resident_ctas()
{
#ifdef QMLP_RESIDENT_CTAS
    return QMLP_RESIDENT_CTAS;
#else
    return 2 * (SmemLayout<Spec>::totalBytes() + 1024) <= 227 * 1024 ? 2 : 1;
#endif
}

template <class Spec, int L>
__device__ __forceinline__ void stage_layer(const LaunchArgs& p, __half* sW, __half* sB)
{
    if constexpr (L < Spec::NUM_LAYERS) {
        using SL = SmemLayout<Spec>;
        constexpr int CIN = Spec::CIN[L], COUT = Spec::COUT[L];
        constexpr int CHUNKS = CIN / 8; // 16-byte chunks per row
        const __half* gW = p.weights + Spec::WOFF[L];
        __half* dW = sW + SL::wOffsetHalfs(L);
        for (int i = threadIdx.x; i < COUT * CHUNKS; i += blockDim.x) {
            const int r = i / CHUNKS, c = i % CHUNKS;
            const uint4 v = *reinterpret_cast<const uint4*>(gW + r * CIN + c * 8);
            *reinterpret_cast<uint4*>(dW + r * SL::wStride(L) + c * 8) = v;
        }
        __half* dB = sB + SL::biasOffset(L);
        for (int i = threadIdx.x; i < COUT; i += blockDim.x)
            dB[i] = Spec::BOFF[L] >= 0 ? p.weights[(Spec::BOFF[L] >= 0 ? Spec::BOFF[L] : 0) + i] : __ushort_as_half(0);
        stage_layer<Spec, L + 1>(p, sW, sB);
    }
}

// ---- encodings (one lane = one point of the warp tile) ---------------------------------------------------------
struct RowReader {
    const float* base; // already offset to the point's row
    long long s1;
    __device__ __forceinline__ float operator()(int c) const { return __ldg(base + c * s1); }
};

struct HalfRowWriter { // one row of the warp's shared-memory tile
    __half* row;
    __device__ __forceinline__ void operator()(int c, float v) const { row[c] = __float2half(v); }
};
struct HalfRowReader {
    const __half* row;
    __device__ __forceinline__ float operator()(int c) const { return __half2float(row[c]); }
};

// ---- line integration ------------------------------------------------------------------------------------------------
// ray start / direction from the input and the parameter interval inside the bounding box
// (IntersectionRayAABB<3>, encoding_line_integration.cuh:27-49: slab test, same operation order)
template <class Enc, class In>
__device__ __forceinline__ void line_ray(const GridP& g, const In& in, float (&start)[3], float (&dir)[3], float& tmin, float& tmax)
{
#pragma unroll
    for (int i = 0; i < 3; ++i) {
        start[i] = in(i + Enc::START);
        dir[i] = in(i + Enc::START + 3);
    }
    const float inv0 = 1.0f / dir[0], inv1 = 1.0f / dir[1], inv2 = 1.0f / dir[2];
    const float t1 = (g.boxMin[0] - start[0]) * inv0, t2 = (g.boxMin[0] + g.boxSize[0] - start[0]) * inv0;
    const float t3 = (g.boxMin[1] - start[1]) * inv1, t4 = (g.boxMin[1] + g.boxSize[1] - start[1]) * inv1;
    const float t5 = (g.boxMin[2] - start[2]) * inv2, t6 = (g.boxMin[2] + g.boxSize[2] - start[2]) * inv2;
    tmin = fmaxf(fmaxf(fminf(t1, t2), fminf(t3, t4)), fminf(t5, t6));
    tmax = fminf(fminf(fmaxf(t1, t2), fmaxf(t3, t4)), fmaxf(t5, t6));
}

// unit-cube position of the sample at parameter t (fma(t, dir, start), then the grid's own box transform)
template <class Enc>
__device__ __forceinline__ void line_sample(const GridP& g, const float (&start)[3], const float (&dir)[3], float t, float (&pos)[3])
{
#pragma unroll
    for (int i = 0; i < 3; ++i) pos[i] = (fmaf(t, dir[i], start[i]) - g.boxMin[i]) * g.boxInvSize[i];
}

template <class Enc, class In, class Out>
__device__ __forceinline__ void line_forward(const GridP& g, const In& in, const Out& out)
{
    float start[3], dir[3], tmin, tmax;
    line_ray<Enc>(g, in, start, dir, tmin, tmax);
    float acc[Enc::NUM_OUT];
#pragma unroll
    for (int i = 0; i < Enc::NUM_OUT; ++i) acc[i] = 0.f;
    for (float t = tmin; t < tmax; t += g.stepsize) {   // encoding_line_integration.cuh:79-85
        float pos[3];
        line_sample<Enc>(g, start, dir, t, pos);
        for (int l = 0; l < Enc::L; ++l) {
            float feat[Enc::F];
            grid_level_forward<3, Enc::F, Enc::HALF_TABLE>(g, g.levels[l], pos, feat);
#pragma unroll
            for (int i = 0; i < Enc::F; ++i) acc[(Enc::CONCAT ? l * Enc::F : 0) + i] += feat[i];
        }
    }
    if constexpr (Enc::AVERAGE) {
        const int steps = static_cast<int>(floorf((tmax - tmin) / g.stepsize));
        if (steps > 0) {
            const float s = 1.0f / static_cast<float>(steps);
#pragma unroll
            for (int i = 0; i < Enc::NUM_OUT; ++i) acc[i] *= s;
        }
    }
#pragma unroll
    for (int i = 0; i < Enc::NUM_OUT; ++i) out(Enc::OUT_OFF + i, acc[i]);
}

// encoding_line_integration.cuh:101-165; the position gradient of a sample goes to the ray start and, times t, to the
// ray direction (the dependence of tmin / tmax on the ray is ignored, as in the reference)
template <class Enc, bool INPUT_GRAD, bool PARAM_GRAD, class In, class AdjOut>
__device__ __forceinline__ void line_adjoint(const GridP& g, const In& in, const AdjOut& adjOut, float* adjInRow, long long aiS1)
{
    const bool paramGrad = PARAM_GRAD && g.grad != nullptr;
    float start[3], dir[3], tmin, tmax;
    line_ray<Enc>(g, in, start, dir, tmin, tmax);
    float scale = 1.0f;
    if constexpr (Enc::AVERAGE) {
        const int steps = static_cast<int>(floorf((tmax - tmin) / g.stepsize));
        scale = steps > 0 ? 1.0f / static_cast<float>(steps) : 1.0f;
    }
    float adjStart[3] = {0.f, 0.f, 0.f}, adjDir[3] = {0.f, 0.f, 0.f};
    for (float t = tmin; t < tmax; t += g.stepsize) {
        float pos[3], adjPos[3] = {0.f, 0.f, 0.f};
        line_sample<Enc>(g, start, dir, t, pos);
        for (int l = 0; l < Enc::L; ++l) {
            float adjF[Enc::F];
#pragma unroll
            for (int i = 0; i < Enc::F; ++i) adjF[i] = scale * adjOut(Enc::OUT_OFF + (Enc::CONCAT ? l * Enc::F : 0) + i);
            if (paramGrad)
                grid_level_adjoint<3, Enc::F, Enc::HALF_TABLE, true, INPUT_GRAD>(g, g.levels[l], pos, adjF, adjPos);
            else if constexpr (INPUT_GRAD)
                grid_level_adjoint<3, Enc::F, Enc::HALF_TABLE, false, true>(g, g.levels[l], pos, adjF, adjPos);
        }
        if constexpr (INPUT_GRAD) {
#pragma unroll
            for (int k = 0; k < 3; ++k) {
                const float a = adjPos[k] * g.boxInvSize[k];
                adjStart[k] += a;
                adjDir[k] += a * t;
            }
        }
    }
    if constexpr (INPUT_GRAD) {
#pragma unroll
        for (int k = 0; k < 3; ++k) {
            adjInRow[(k + Enc::START) * aiS1] += adjStart[k];
            adjInRow[(k + Enc::START + 3) * aiS1] += adjDir[k];
        }
    }
}

template <class Spec, int E, class Out>
__device__ __forceinline__ void encode_point(const LaunchArgs& p, const RowReader& in, const Out& out)
{
    if constexpr (E < Spec::NUM_ENCODINGS) {
        using Enc = typename Spec::template Enc<E>;
        if constexpr (Enc::IS_LINE) {
            line_forward<Enc>(p.grids[Enc::SLOT], in, out);
        } else if constexpr (!Enc::IS_GRID) {
            // src_cpp/include/qmlp/kernels/encoding_identity.cuh:16-25
#pragma unroll
            for (int i = 0; i < Enc::N; ++i) out(Enc::OUT_OFF + i, in(i + Enc::START));
        } else {
            const GridP& g = p.grids[Enc::SLOT];
            float pos[Enc::D];
            grid_position<Enc::D, Enc::START>(g, in, pos);
            if constexpr (Enc::CONCAT) {
#pragma unroll 2
                for (int l = 0; l < Enc::L; ++l) {
                    float feat[Enc::F];
                    grid_level_forward<Enc::D, Enc::F, Enc::HALF_TABLE>(g, g.levels[l], pos, feat);
#pragma unroll
                    for (int i = 0; i < Enc::F; ++i) out(Enc::OUT_OFF + l * Enc::F + i, feat[i]);
                }
            } else {
                // "add": the reference accumulates the half outputs level by level (encoding_hashgrid.cuh:330-335)
                float acc[Enc::F];
#pragma unroll
                for (int i = 0; i < Enc::F; ++i) acc[i] = 0.f;
                for (int l = 0; l < Enc::L; ++l) {
                    float feat[Enc::F];
                    grid_level_forward<Enc::D, Enc::F, Enc::HALF_TABLE>(g, g.levels[l], pos, feat);
#pragma unroll
                    for (int i = 0; i < Enc::F; ++i) acc[i] += feat[i];
                }
#pragma unroll
                for (int i = 0; i < Enc::F; ++i) out(Enc::OUT_OFF + i, acc[i]);
            }
        }
        encode_point<Spec, E + 1, Out>(p, in, out);
    }
}

// ---- layer-0 operand from level-major feature planes ---------------------------------------------------------------
// (written by encode_planes_kernel, kernels/grid_planes.cuh: plane of channel c = planes + planeStride * c, F halfs per
// point for the F channels of one grid level, N halfs per point for an identity encoding)
struct HalfRowPlaneWriter { // one row of the warp's shared-memory tile, fed with halfs
    __half* row;
    __device__ __forceinline__ void half(int c, __half v) const { row[c] = v; }
    __device__ __forceinline__ void half2(int c, uint32_t v) const { *reinterpret_cast<uint32_t*>(row + c) = v; }
};

// layer-0 operand row of one point from the planes (Out writes halfs: out.half(channel, value)).
// All plane values of an encoding are fetched into registers before the first one is written: the writes go to shared
// memory through a generic pointer, so a load placed after a write could not be moved above it, and the 16 loads of
// configuration 5 would run one memory latency after the other (measured: 22 700 cycles per tile instead of ~5 000).
template <class Spec, int E, class Out>
__device__ __forceinline__ void read_planes_point(const LaunchArgs& p, long long local, const Out& out)
{
    if constexpr (E < Spec::NUM_ENCODINGS) {
        using Enc = typename Spec::template Enc<E>;
        if constexpr (!Enc::IS_GRID) {
            const __half* src = p.planes + p.planeStride * Enc::OUT_OFF + local * Enc::N;
            const bool ok = scratch_ok(p, src - p.planes, Enc::N, p.planeHalfs, STATUS_PLANES);
            __half v[Enc::N];
#pragma unroll
            for (int i = 0; i < Enc::N; ++i) v[i] = ok ? __ldg(src + i) : __ushort_as_half(0);
#pragma unroll
            for (int i = 0; i < Enc::N; ++i) out.half(Enc::OUT_OFF + i, v[i]);
        } else {
            constexpr int GROUPS = Enc::CONCAT ? Enc::L : 1;
            constexpr int F = Enc::F;
            const __half* base = p.planes + p.planeStride * Enc::OUT_OFF + local * F;
            if constexpr (BOUNDS_CHECK) {
                // the planes of this encoding's levels: first and last one read below
                if (!scratch_ok(p, base - p.planes, F, p.planeHalfs, STATUS_PLANES) ||
                    !scratch_ok(p, (base - p.planes) + p.planeStride * ((GROUPS - 1) * F), F, p.planeHalfs, STATUS_PLANES)) {
#pragma unroll
                    for (int i = 0; i < GROUPS * F; ++i) out.half(Enc::OUT_OFF + i, __ushort_as_half(0));
                    read_planes_point<Spec, E + 1, Out>(p, local, out);
                    return;
                }
            }
            if constexpr (F == 2) {
                uint32_t v[GROUPS];
#pragma unroll
                for (int l = 0; l < GROUPS; ++l) v[l] = ldg_nc_u32(base + p.planeStride * (l * F));
#pragma unroll
                for (int l = 0; l < GROUPS; ++l) out.half2(Enc::OUT_OFF + l * F, v[l]);
            } else if constexpr (F == 4) {
                uint2 v[GROUPS];
#pragma unroll
                for (int l = 0; l < GROUPS; ++l) v[l] = ldg_nc_u64(base + p.planeStride * (l * F));
#pragma unroll
                for (int l = 0; l < GROUPS; ++l) {
                    out.half2(Enc::OUT_OFF + l * F, v[l].x);
                    out.half2(Enc::OUT_OFF + l * F + 2, v[l].y);
                }
            } else if constexpr (F == 8) {
                uint4 v[GROUPS];
#pragma unroll
                for (int l = 0; l < GROUPS; ++l) v[l] = ldg_nc_u128(base + p.planeStride * (l * F));
#pragma unroll
                for (int l = 0; l < GROUPS; ++l) {
                    out.half2(Enc::OUT_OFF + l * F, v[l].x);
                    out.half2(Enc::OUT_OFF + l * F + 2, v[l].y);
                    out.half2(Enc::OUT_OFF + l * F + 4, v[l].z);
                    out.half2(Enc::OUT_OFF + l * F + 6, v[l].w);
                }
            } else {
                __half v[GROUPS * F];
#pragma unroll
                for (int l = 0; l < GROUPS; ++l)
#pragma unroll
                    for (int i = 0; i < F; ++i) v[l * F + i] = __ldg(base + p.planeStride * (l * F) + i);
#pragma unroll
                for (int i = 0; i < GROUPS * F; ++i) out.half(Enc::OUT_OFF + i, v[i]);
            }
        }
        read_planes_point<Spec, E + 1, Out>(p, local, out);
    }
}

// ---- forward layer chain -------------------------------------------------------------------------------------
// MODE 0: inference, 1: forward with stash, 2: forward with stash + L2 loss gradient instead of the output
template <class Spec, int L, int MODE>
__device__ __forceinline__ void forward_layers(const LaunchArgs& p, const __half* sW, const __half* sB,
                                               uint32_t (&aIn)[MT][Spec::CIN[L] / 16][4], long long rowBase, long long n32,
                                               float& lossAcc)
{
    using SL = SmemLayout<Spec>;
    using Act = typename Spec::template Act<L>;
    constexpr int CIN = Spec::CIN[L], COUT = Spec::COUT[L];
    constexpr int KT = CIN / 16, NC = COUT / 16;
    constexpr bool LAST = (L == Spec::NUM_LAYERS - 1);
    constexpr int WS = SL::wStride(L);
    const int lane = threadIdx.x & 31;
    const int r = lane >> 2, q = lane & 3;
    const __half* w = sW + SL::wOffsetHalfs(L);
    const __half* bias = sB + SL::biasOffset(L);
    constexpr bool BIAS = Spec::BOFF[L] >= 0;
    // ldmatrix lane address of the B fragments: two n8 tiles x (k 0-7, k 8-15)
    const uint32_t wAddr = smem_u32(w + ((lane & 7) + ((lane >> 4) << 3)) * WS + ((lane >> 3) & 1) * 8);

    uint32_t aOut[MT][LAST ? 1 : NC][4];
#pragma unroll
    for (int j = 0; j < NC; ++j) {
        if constexpr (LAST) {
            if (j * 16 >= Spec::NUM_OUTPUTS) continue; // padded output channels are never read
        }
        float acc[MT][2][4];
#pragma unroll
        for (int m = 0; m < MT; ++m)
#pragma unroll
            for (int h = 0; h < 2; ++h)
#pragma unroll
                for (int e = 0; e < 4; ++e) acc[m][h][e] = 0.f;
#pragma unroll
        for (int k = 0; k < KT; ++k) {
            uint32_t b[4];
            ldmatrix_x4(b, wAddr + (j * 16 * WS + k * 16) * 2);
#pragma unroll
            for (int m = 0; m < MT; ++m) {
                mma16816(acc[m][0], aIn[m][k], b[0], b[1]);
                mma16816(acc[m][1], aIn[m][k], b[2], b[3]);
            }
        }
#pragma unroll
        for (int m = 0; m < MT; ++m) {
            __half2 pre[2][2]; // [h][row r | row r + 8]
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                pre[h][0] = __floats2half2_rn(acc[m][h][0], acc[m][h][1]);
                pre[h][1] = __floats2half2_rn(acc[m][h][2], acc[m][h][3]);
                if constexpr (BIAS) {
                    // the fp32 accumulator is rounded to half first, then the (half) bias is added
                    const __half2 b2 = *reinterpret_cast<const __half2*>(bias + j * 16 + h * 8 + q * 2);
                    pre[h][0] = __hadd2(pre[h][0], b2);
                    pre[h][1] = __hadd2(pre[h][1], b2);
                }
            }
            const long long row0 = rowBase + m * 16 + r;
            if constexpr (MODE >= 1) {
                // pre-activation stash (N32, COUT) per layer (reference: kernels/layer.cuh:156-163) in 8 x 8 blocks
                // (stash_block): a register of the warp is one 128-byte line
                __half* st = p.fwdTmp + n32 * SL::preOffset(L) + (r * 8 + q * 2);
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const long long lo = stash_block(rowBase, COUT, m * 2, j * 2 + h), hi = stash_block(rowBase, COUT, m * 2 + 1, j * 2 + h);
                    if (row0 < p.numel && scratch_ok(p, (st - p.fwdTmp) + lo, 2, p.fwdTmpHalfs, STATUS_STASH))
                        *reinterpret_cast<__half2*>(st + lo) = pre[h][0];
                    if (row0 + 8 < p.numel && scratch_ok(p, (st - p.fwdTmp) + hi, 2, p.fwdTmpHalfs, STATUS_STASH))
                        *reinterpret_cast<__half2*>(st + hi) = pre[h][1];
                }
            }
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const int col = j * 16 + h * 8 + q * 2;
                const __half2 lo = pre[h][0], hi = pre[h][1];
                const __half2 zlo = act_forward2<Act>(lo, col), zhi = act_forward2<Act>(hi, col);
                if constexpr (!LAST) {
                    aOut[m][j][h * 2 + 0] = h2_as_u32(zlo);
                    aOut[m][j][h * 2 + 1] = h2_as_u32(zhi);
                } else {
                    // first NUM_OUTPUTS channels -> fp32 (kernels/network_forward.cuh:103-111)
                    const float2 flo = __half22float2(zlo), fhi = __half22float2(zhi);
                    const float v[4] = {flo.x, flo.y, fhi.x, fhi.y};
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const long long row = row0 + (e >> 1) * 8;
                        const int c = col + (e & 1);
                        if (c < Spec::NUM_OUTPUTS && row < p.numel) { // the row is the same for the four lanes of a quad
                            if constexpr (MODE == 2) {
                                const float d = v[e] - __ldg(p.target + row * p.tS0 + c * p.tS1);
                                lossAcc += d * d;
                                p.output[row * p.outS0 + c * p.outS1] = p.lossScale * d;
                            } else {
                                p.output[row * p.outS0 + c * p.outS1] = v[e];
                            }
                        }
                    }
                }
            }
        }
    }
    if constexpr (!LAST) forward_layers<Spec, L + 1, MODE>(p, sW, sB, aOut, rowBase, n32, lossAcc);
}

// MODE_ bit 2 (value 4): the encodings were computed by encode_planes_kernel; layer 0 reads the feature planes
template <class Spec, int MODE_>
__global__ void __launch_bounds__(Spec::WARPS * 32, resident_ctas<Spec>())
fused_forward_kernel(const __grid_constant__ LaunchArgs p)
{
    constexpr int MODE = MODE_ & 3;
    constexpr bool FROM_PLANES = (MODE_ & 4) != 0;
    using SL = SmemLayout<Spec>;
    extern __shared__ __align__(16) unsigned char smem[];
    __half* sW = reinterpret_cast<__half*>(smem);
    __half* sB = reinterpret_cast<__half*>(smem + SL::biasStartBytes());
    stage_layer<Spec, 0>(p, sW, sB);
    __syncthreads();

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    __half* tile = reinterpret_cast<__half*>(smem + SL::tileStartBytes() + warp * SL::tileBytesPerWarp());
    constexpr int TS = SL::tileStride();
    constexpr int CIN0 = Spec::CIN[0];
    const long long n32 = (p.numel + 31) / 32 * 32;
    const long long numTiles = n32 / TILE_POINTS;
    float lossAcc = 0.f;

    for (long long t = static_cast<long long>(blockIdx.x) * Spec::WARPS + warp; t < numTiles;
         t += static_cast<long long>(gridDim.x) * Spec::WARPS) {
        const long long rowBase = t * TILE_POINTS;
        const long long myRow = rowBase + lane;
        __half* row = tile + lane * TS;
        // encodings; padding channels and invalid tail points are zero (kernels/network_forward.cuh:67-89)
        if (myRow < p.numel) {
            if constexpr (FROM_PLANES) {
                read_planes_point<Spec, 0>(p, myRow, HalfRowPlaneWriter{row});
            } else {
                RowReader in{p.input + myRow * p.inS0, p.inS1};
                encode_point<Spec, 0>(p, in, HalfRowWriter{row});
            }
#pragma unroll
            for (int c = Spec::ENC_CHANNELS; c < CIN0; ++c) row[c] = __ushort_as_half(0);
        } else {
#pragma unroll
            for (int c = 0; c < CIN0; c += 8) *reinterpret_cast<uint4*>(row + c) = make_uint4(0, 0, 0, 0);
        }
        __syncwarp();
        if constexpr (MODE >= 1) {
            // stash the encoded input: the layer-0 weight gradient reads it instead of re-running the encodings
            constexpr int CH = CIN0 / 8;
            __half* st = p.fwdTmp; // offset 0
            for (int i = lane; i < TILE_POINTS * CH; i += 32) {
                const int rr = i / CH, cc = i % CH;
                if (rowBase + rr < p.numel && scratch_ok(p, (rowBase + rr) * CIN0 + cc * 8, 8, p.fwdTmpHalfs, STATUS_STASH))
                    *reinterpret_cast<uint4*>(st + (rowBase + rr) * CIN0 + cc * 8) = *reinterpret_cast<const uint4*>(tile + rr * TS + cc * 8);
            }
        }
        uint32_t a0[MT][CIN0 / 16][4];
#pragma unroll
        for (int m = 0; m < MT; ++m)
#pragma unroll
            for (int k = 0; k < CIN0 / 16; ++k)
                ldmatrix_x4(a0[m][k], smem_u32(tile + (m * 16 + (lane & 15)) * TS + k * 16 + (lane >> 4) * 8));
        __syncwarp();
        forward_layers<Spec, 0, MODE>(p, sW, sB, a0, rowBase, n32, lossAcc);
    }
    if constexpr (MODE == 2) {
        if (p.lossSum != nullptr) {
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) lossAcc += __shfl_xor_sync(0xffffffffu, lossAcc, o);
            if (lane == 0 && lossAcc != 0.f) atomicAdd(p.lossSum, lossAcc);
        }
    }
}

// ---- adjoint -------------------------------------------------------------------------------------------------
template <class Spec, int E, bool INPUT_GRAD, bool PARAM_GRAD, class AdjOut>
__device__ __forceinline__ void encode_adjoint_point(const LaunchArgs& p, const RowReader& in, const AdjOut& adjOut,
                                                     float* adjInRow, long long aiS1)
{
    if constexpr (E < Spec::NUM_ENCODINGS) {
        using Enc = typename Spec::template Enc<E>;
        if constexpr (Enc::IS_LINE) {
            line_adjoint<Enc, INPUT_GRAD, PARAM_GRAD>(p.grids[Enc::SLOT], in, adjOut, adjInRow, aiS1);
        } else if constexpr (!Enc::IS_GRID) {
            // src_cpp/include/qmlp/kernels/encoding_identity.cuh:27-38
            if constexpr (INPUT_GRAD) {
#pragma unroll
                for (int i = 0; i < Enc::N; ++i) adjInRow[(i + Enc::START) * aiS1] += adjOut(Enc::OUT_OFF + i);
            }
        } else {
            const GridP& g = p.grids[Enc::SLOT];
            const bool paramGrad = PARAM_GRAD && g.grad != nullptr;
            float pos[Enc::D], adjPos[Enc::D];
            grid_position<Enc::D, Enc::START>(g, in, pos);
#pragma unroll
            for (int k = 0; k < Enc::D; ++k) adjPos[k] = 0.f;
            for (int l = 0; l < Enc::L; ++l) {
                float adjF[Enc::F];
#pragma unroll
                for (int i = 0; i < Enc::F; ++i) adjF[i] = adjOut(Enc::OUT_OFF + (Enc::CONCAT ? l * Enc::F : 0) + i);
                if (paramGrad)
                    grid_level_adjoint<Enc::D, Enc::F, Enc::HALF_TABLE, true, INPUT_GRAD>(g, g.levels[l], pos, adjF, adjPos);
                else if constexpr (INPUT_GRAD)
                    grid_level_adjoint<Enc::D, Enc::F, Enc::HALF_TABLE, false, true>(g, g.levels[l], pos, adjF, adjPos);
            }
            if constexpr (INPUT_GRAD) {
                // encoding_hashgrid.cuh:414-421
#pragma unroll
                for (int k = 0; k < Enc::D; ++k) adjInRow[(k + Enc::START) * aiS1] += adjPos[k] * g.boxInvSize[k];
            }
        }
        encode_adjoint_point<Spec, E + 1, INPUT_GRAD, PARAM_GRAD, AdjOut>(p, in, adjOut, adjInRow, aiS1);
    }
}

// Adjoint of the grid features of one point -> level-major planes (one plane per grid level of a concatenating grid,
// one per adding grid; plane of channel c0 = planes + planeStride * c0, F halfs per point): what
// scatter_planes_kernel consumes. `row` is the point's row of adjoint features in the warp's shared tile.
template <class Spec, int E>
__device__ __forceinline__ void write_adjoint_planes(const LaunchArgs& p, long long point, const __half* row)
{
    if constexpr (E < Spec::NUM_ENCODINGS) {
        using Enc = typename Spec::template Enc<E>;
        if constexpr (Enc::IS_GRID) {
            constexpr int GROUPS = Enc::CONCAT ? Enc::L : 1;
#pragma unroll
            for (int l = 0; l < GROUPS; ++l) {
                constexpr int F = Enc::F;
                const int c0 = Enc::OUT_OFF + l * F;
                __half* dst = p.planes + p.planeStride * c0 + point * F;
                if (!scratch_ok(p, dst - p.planes, F, p.planeHalfs, STATUS_PLANES)) continue;
                if constexpr (F % 2 == 0) {
                    uint32_t w[F / 2];
#pragma unroll
                    for (int i = 0; i < F / 2; ++i)
                        w[i] = static_cast<uint32_t>(__half_as_ushort(row[c0 + 2 * i])) |
                               (static_cast<uint32_t>(__half_as_ushort(row[c0 + 2 * i + 1])) << 16);
                    if constexpr (F == 2) *reinterpret_cast<uint32_t*>(dst) = w[0];
                    else if constexpr (F == 4) *reinterpret_cast<uint2*>(dst) = make_uint2(w[0], w[1]);
                    else if constexpr (F == 8) *reinterpret_cast<uint4*>(dst) = make_uint4(w[0], w[1], w[2], w[3]);
                    else {
#pragma unroll
                        for (int i = 0; i < F / 2; ++i) reinterpret_cast<uint32_t*>(dst)[i] = w[i];
                    }
                } else {
#pragma unroll
                    for (int i = 0; i < F; ++i) dst[i] = row[c0 + i];
                }
            }
        }
        write_adjoint_planes<Spec, E + 1>(p, point, row);
    }
}

// FLAGS: FLAG_GRAD_INPUT | FLAG_GRAD_WEIGHTS | FLAG_GRAD_ENCODINGS [| FLAG_SPLIT_SCATTER]
template <class Spec, int L, int FLAGS>
__device__ __forceinline__ void backward_layers(const LaunchArgs& p, const __half* sW,
                                                uint32_t (&adj)[MT][Spec::COUT[L] / 16][4], long long rowBase,
                                                long long n32, __half* tile)
{
    using SL = SmemLayout<Spec>;
    using Act = typename Spec::template Act<L>;
    constexpr int CIN = Spec::CIN[L], COUT = Spec::COUT[L];
    constexpr int KT = COUT / 16, NC = CIN / 16;
    constexpr int WS = SL::wStride(L);
    constexpr bool NEED_ENC = (FLAGS & (FLAG_GRAD_INPUT | FLAG_GRAD_ENCODINGS)) != 0;
    const int lane = threadIdx.x & 31;
    const int r = lane >> 2, q = lane & 3;

    // delta = Act'(pre) * adj, in place (kernels/layer.cuh:216-229), pre-activations read back in fragment layout
    const __half* pre = p.fwdTmp + n32 * SL::preOffset(L);
    __half* dl = p.adjTmp + n32 * SL::deltaOffset(L);
    // All pre-activations of a row tile are requested before the first delta is stored: the stores go to memory the
    // compiler cannot tell apart from the stash, so a load placed after one would wait for it to issue, and the loads
    // would run one memory latency after the other.
#pragma unroll
    for (int m = 0; m < MT; ++m) {
        uint32_t x[KT][4];
#pragma unroll
        for (int k = 0; k < KT; ++k)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const long long row = rowBase + m * 16 + r + (e & 1) * 8;
                const long long at = stash_block(rowBase, COUT, m * 2 + (e & 1), k * 2 + (e >> 1)) + (r * 8 + q * 2);
                const bool ok = row < p.numel && scratch_ok(p, (pre - p.fwdTmp) + at, 2, p.fwdTmpHalfs, STATUS_STASH);
                x[k][e] = ok ? __ldg(reinterpret_cast<const unsigned int*>(pre + at)) : 0u;
            }
#pragma unroll
        for (int k = 0; k < KT; ++k)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const long long row = rowBase + m * 16 + r + (e & 1) * 8;
                const int col = k * 16 + (e >> 1) * 8 + q * 2;
                const long long at = stash_block(rowBase, COUT, m * 2 + (e & 1), k * 2 + (e >> 1)) + (r * 8 + q * 2);
                const __half2 d = act_adjoint2<Act>(u32_as_h2(x[k][e]), u32_as_h2(adj[m][k][e]), col);
                adj[m][k][e] = h2_as_u32(d);
                if constexpr ((FLAGS & FLAG_GRAD_WEIGHTS) != 0) {
                    if (row < p.numel && scratch_ok(p, (dl - p.adjTmp) + at, 2, p.adjTmpHalfs, STATUS_STASH))
                        *reinterpret_cast<__half2*>(dl + at) = d;
                }
            }
    }

    if constexpr (L > 0 || NEED_ENC) {
        // adjIn (points x CIN) = delta (points x COUT) * W (COUT x CIN): B fragments by transposing ldmatrix
        const __half* w = sW + SL::wOffsetHalfs(L);
        const uint32_t wAddr = smem_u32(w + ((lane & 7) + ((lane >> 3) & 1) * 8) * WS + (lane >> 4) * 8);
        uint32_t adjIn[MT][NC][4];
#pragma unroll
        for (int j = 0; j < NC; ++j) {
            float acc[MT][2][4];
#pragma unroll
            for (int m = 0; m < MT; ++m)
#pragma unroll
                for (int h = 0; h < 2; ++h)
#pragma unroll
                    for (int e = 0; e < 4; ++e) acc[m][h][e] = 0.f;
#pragma unroll
            for (int k = 0; k < KT; ++k) {
                uint32_t b[4];
                ldmatrix_x4_trans(b, wAddr + (k * 16 * WS + j * 16) * 2);
#pragma unroll
                for (int m = 0; m < MT; ++m) {
                    mma16816(acc[m][0], adj[m][k], b[0], b[1]);
                    mma16816(acc[m][1], adj[m][k], b[2], b[3]);
                }
            }
#pragma unroll
            for (int m = 0; m < MT; ++m)
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    adjIn[m][j][h * 2 + 0] = h2_as_u32(__floats2half2_rn(acc[m][h][0], acc[m][h][1]));
                    adjIn[m][j][h * 2 + 1] = h2_as_u32(__floats2half2_rn(acc[m][h][2], acc[m][h][3]));
                }
        }
        if constexpr (L > 0) {
            backward_layers<Spec, L - 1, FLAGS>(p, sW, adjIn, rowBase, n32, tile);
        } else {
            // adjoint of the encoded features -> shared tile, then one lane per point runs the encoding adjoints
            constexpr int TS = SL::tileStride();
#pragma unroll
            for (int m = 0; m < MT; ++m)
#pragma unroll
                for (int j = 0; j < NC; ++j)
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int rr = m * 16 + r + (e & 1) * 8;
                        const int cc = j * 16 + (e >> 1) * 8 + q * 2;
                        *reinterpret_cast<uint32_t*>(tile + rr * TS + cc) = adjIn[m][j][e];
                    }
            __syncwarp();
            const long long myRow = rowBase + lane;
            if (myRow < p.numel) {
                if constexpr ((FLAGS & FLAG_SPLIT_SCATTER) != 0) {
                    write_adjoint_planes<Spec, 0>(p, myRow, tile + lane * TS);
                } else {
                    RowReader in{p.input + myRow * p.inS0, p.inS1};
                    float* adjInRow = (FLAGS & FLAG_GRAD_INPUT) ? p.adjInput + myRow * p.aiS0 : nullptr;
                    encode_adjoint_point<Spec, 0, (FLAGS & FLAG_GRAD_INPUT) != 0, (FLAGS & FLAG_GRAD_ENCODINGS) != 0>(
                        p, in, HalfRowReader{tile + lane * TS}, adjInRow, p.aiS1);
                }
            }
            __syncwarp();
        }
    }
}

template <class Spec, int FLAGS>
__global__ void __launch_bounds__(Spec::WARPS * 32, resident_ctas<Spec>())
fused_backward_kernel(const __grid_constant__ LaunchArgs p)
{
    using SL = SmemLayout<Spec>;
    extern __shared__ __align__(16) unsigned char smem[];
    __half* sW = reinterpret_cast<__half*>(smem);
    __half* sB = reinterpret_cast<__half*>(smem + SL::biasStartBytes());
    stage_layer<Spec, 0>(p, sW, sB);
    __syncthreads();

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int r = lane >> 2, q = lane & 3;
    __half* tile = reinterpret_cast<__half*>(smem + SL::tileStartBytes() + warp * SL::tileBytesPerWarp());
    constexpr int LL = Spec::NUM_LAYERS - 1;
    constexpr int KT = Spec::COUT[LL] / 16;
    const long long n32 = (p.numel + 31) / 32 * 32;
    const long long numTiles = n32 / TILE_POINTS;

    for (long long t = static_cast<long long>(blockIdx.x) * Spec::WARPS + warp; t < numTiles;
         t += static_cast<long long>(gridDim.x) * Spec::WARPS) {
        const long long rowBase = t * TILE_POINTS;
        // dL/dout (fp32, N x NUM_OUTPUTS) -> half fragments, zero padded (kernels/network_backward.cuh:67-80)
        uint32_t adj[MT][KT][4];
#pragma unroll
        for (int m = 0; m < MT; ++m)
#pragma unroll
            for (int k = 0; k < KT; ++k)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const long long row = rowBase + m * 16 + r + (e & 1) * 8;
                    const int col = k * 16 + (e >> 1) * 8 + q * 2;
                    float v0 = 0.f, v1 = 0.f;
                    if (row < p.numel) {
                        if (col < Spec::NUM_OUTPUTS) v0 = __ldg(p.adjOutput + row * p.aoS0 + col * p.aoS1);
                        if (col + 1 < Spec::NUM_OUTPUTS) v1 = __ldg(p.adjOutput + row * p.aoS0 + (col + 1) * p.aoS1);
                    }
                    adj[m][k][e] = h2_as_u32(__floats2half2_rn(v0, v1));
                }
        backward_layers<Spec, LL, FLAGS>(p, sW, adj, rowBase, n32, tile);
    }
}

// ---- weight / bias gradient: split-batch tensor-core GEMM -------------------------------------------------------
// dW_l (COUT x CIN) += sum_n delta_l[n,:]^T * a_{l-1}[n,:],  db_l += sum_n delta_l[n,:]
// (math of tests_cpp/test_against_eigen2.cpp:187-200; replaces the single-block WeightUpdateSingleBlockKernel,
// src_cpp/include/qmlp/kernels/network_weight_update_block.cuh:356-494). a_{l-1} is recomputed from the stashed
// pre-activation (or is the stashed encoded input for l == 0). Each CTA works on one layer (WgradSplit) and strides
// over 64-point slabs; partial sums are added to the fp32 gradient vector with red.global.add.
constexpr int WG_SLAB = 64;
constexpr int WG_WARPS = 8;

template <class Spec>
struct WgradSmem {
    __host__ __device__ static constexpr int maxCout() { int m = 0; for (int i = 0; i < Spec::NUM_LAYERS; ++i) m = Spec::COUT[i] > m ? Spec::COUT[i] : m; return m; }
    __host__ __device__ static constexpr int maxCin() { int m = 0; for (int i = 0; i < Spec::NUM_LAYERS; ++i) m = Spec::CIN[i] > m ? Spec::CIN[i] : m; return m; }
    __host__ __device__ static constexpr int stageBytes() { return WG_SLAB * ((maxCout() + 8) + (maxCin() + 8)) * 2; }
    // Slabs in flight per CTA. The kernel does little work per byte, so what it reaches is set by how many bytes each
    // SM keeps requested: with two buffers a CTA waits out one full memory latency per slab (config 4: 2.9 TB/s).
    // As many stages as two CTAs per SM have shared memory for, at most four.
    __host__ __device__ static constexpr int stages()
    {
        int st = (224 * 1024 / 2) / stageBytes();
        return st > 4 ? 4 : (st < 2 ? 2 : st);
    }
    __host__ __device__ static constexpr int bytes() { return stages() * stageBytes(); }
};

// CTAs of the one-dimensional grid are dealt to the layers in proportion to the bytes a layer reads per point
// (delta row + input row): the kernel is bound by that traffic, and an equal share per layer leaves the narrow layers'
// CTAs idle while the wide ones finish (config 4: 176 : 192 : 80 : 32).
template <class Spec>
struct WgradSplit {
    __host__ __device__ static constexpr int weight(int l) { return Spec::CIN[l] + Spec::COUT[l]; }
    __host__ __device__ static constexpr int total()
    {
        int t = 0;
        for (int i = 0; i < Spec::NUM_LAYERS; ++i) t += weight(i);
        return t;
    }
    // smallest grid that gives every layer at least one CTA
    __host__ __device__ static constexpr int minCtas()
    {
        int m = weight(0);
        for (int i = 1; i < Spec::NUM_LAYERS; ++i) m = weight(i) < m ? weight(i) : m;
        return (total() + m - 1) / m;
    }
    __host__ __device__ static constexpr long long prefix(int l)
    {
        long long s = 0;
        for (int i = 0; i < l; ++i) s += weight(i);
        return s;
    }
    // first CTA of layer L in a grid of `ctas` (layer L owns [begin<L>, begin<L + 1>))
    template <int L>
    __host__ __device__ static int begin(int ctas)
    {
        constexpr long long before = prefix(L);
        constexpr long long all = total();
        return static_cast<int>(before * ctas / all);
    }
};

// `cta` of `ctas`: this CTA's rank among the CTAs working on layer L
template <class Spec, int L>
__device__ __forceinline__ void wgrad_layer(const LaunchArgs& p, unsigned char* smem, int cta, int ctas)
{
    using SL = SmemLayout<Spec>;
    constexpr int CIN = Spec::CIN[L], COUT = Spec::COUT[L];
    constexpr int BS = CIN + 8;                         // smem row stride of the row-major encoded input (halfs)
    constexpr int NBLK = (COUT / 16) * (CIN / 16);      // 16x16 output blocks
    constexpr int WB = NBLK >= 8 ? 8 : NBLK >= 4 ? 4 : NBLK >= 2 ? 2 : 1; // warps across blocks
    constexpr int KW = WG_WARPS / WB;                   // warps across the k16 steps of a slab
    constexpr int PB = (NBLK + WB - 1) / WB;            // blocks per warp
    constexpr bool BIAS = Spec::BOFF[L] >= 0;

    // Points per pipeline stage of this layer: as many as the stage (sized for 64 points of the widest layer) holds, so
    // that every layer moves about the same number of bytes per stage. With 64 points everywhere a 16 -> 16 layer
    // spent its time on the two barriers per 4 KB slab (config 4: its CTAs finished last).
    constexpr int A_STRIDE = L == 0 ? BS : CIN;         // the blocked operands need no padding
    constexpr int SLAB_MAX = WgradSmem<Spec>::stageBytes() / ((COUT + A_STRIDE) * 2) / 64 * 64;
    constexpr int SLAB = SLAB_MAX > 512 ? 512 : SLAB_MAX;
    static_assert(SLAB >= WG_SLAB, "a stage holds at least 64 points of every layer");
    constexpr int KSTEPS = SLAB / 16;
    constexpr int ST = WgradSmem<Spec>::stages();
    constexpr int STAGE_HALFS = SLAB * (COUT + A_STRIDE);
    __half* const sDbase = reinterpret_cast<__half*>(smem);            // stage s: [SLAB x COUT | SLAB x A_STRIDE]
    __half* const sAbase = sDbase + SLAB * COUT;

    const long long n32 = (p.numel + 31) / 32 * 32;
    const __half* gD = p.adjTmp + n32 * SL::deltaOffset(L);
    const __half* gA = L == 0 ? p.fwdTmp : p.fwdTmp + n32 * SL::preOffset(L > 0 ? L - 1 : 0);
    const long long numSlabs = (p.numel + SLAB - 1) / SLAB;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int wb = warp % WB, wk = warp / WB;

    float acc[PB][2][4];
    float accB[PB][4];
#pragma unroll
    for (int b = 0; b < PB; ++b) {
#pragma unroll
        for (int e = 0; e < 4; ++e) { acc[b][0][e] = 0.f; acc[b][1][e] = 0.f; accB[b][e] = 0.f; }
    }

    auto load_slab = [&](long long slab, int buf) {
        const long long row0 = slab * SLAB;
        constexpr int DCH = COUT / 8, ACH = CIN / 8;
        // 16-byte pieces (one point, 8 channels). Deltas and pre-activations lie in 8 x 8 blocks (stash_block) and are
        // copied as they are: in shared memory an 8 x 8 block is then one 128-byte line, which is exactly what one
        // ldmatrix matrix reads (no bank conflicts, no padding). The encoded input (L == 0) is row-major with padded rows.
        for (int i = threadIdx.x; i < SLAB * DCH; i += WG_WARPS * 32) {
            const int rr = (i / (32 * DCH)) * 32 + (i % 32);        // the point of piece i (storage order)
            const bool ok = row0 + rr < p.numel && scratch_ok(p, (gD - p.adjTmp) + row0 * COUT + i * 8, 8, p.adjTmpHalfs, STATUS_STASH);
            cp_async16(smem_u32(sDbase + buf * STAGE_HALFS + i * 8), gD + (ok ? row0 * COUT + i * 8 : 0), ok);
        }
        for (int i = threadIdx.x; i < SLAB * ACH; i += WG_WARPS * 32) {
            if constexpr (L == 0) {
                const int rr = i / ACH, cc = i % ACH;
                const bool ok = row0 + rr < p.numel && scratch_ok(p, (gA - p.fwdTmp) + (row0 + rr) * CIN + cc * 8, 8, p.fwdTmpHalfs, STATUS_STASH);
                cp_async16(smem_u32(sAbase + buf * STAGE_HALFS + rr * BS + cc * 8), gA + (ok ? row0 + rr : 0) * CIN + cc * 8, ok);
            } else {
                const int rr = (i / (32 * ACH)) * 32 + (i % 32);
                const bool ok = row0 + rr < p.numel && scratch_ok(p, (gA - p.fwdTmp) + row0 * CIN + i * 8, 8, p.fwdTmpHalfs, STATUS_STASH);
                cp_async16(smem_u32(sAbase + buf * STAGE_HALFS + i * 8), gA + (ok ? row0 * CIN + i * 8 : 0), ok);
            }
        }
    };

    long long slab = cta;
    int buf = 0;
#pragma unroll
    for (int i = 0; i < ST - 1; ++i) {   // one commit group per slab, empty past the end
        if (slab + static_cast<long long>(i) * ctas < numSlabs) load_slab(slab + static_cast<long long>(i) * ctas, i);
        cp_async_commit();
    }
    for (; slab < numSlabs; slab += ctas) {
        // the buffer refilled here was read in the previous iteration, which ended with __syncthreads()
        const long long next = slab + static_cast<long long>(ST - 1) * ctas;
        if (next < numSlabs) load_slab(next, (buf + ST - 1) % ST);
        cp_async_commit();
        cp_async_wait<ST - 1>();
        __syncthreads();
        const __half* d = sDbase + buf * STAGE_HALFS;
        const __half* a = sAbase + buf * STAGE_HALFS;
        // B fragment (k = point, n = cin) of column block nb: transposing ldmatrix of the (point, cin) tile, then
        // a_{l-1} = Act_{l-1}(stashed pre-activation) on it
        // offset of (point row, 8-channel column block cb) of a slab in the blocked layout
        auto blocked = [](int row, int cb, int channels) {
            return (row >> 5) * 32 * channels + ((cb * 4 + ((row & 31) >> 3)) * 64) + (row & 7) * 8;
        };
        auto load_b = [&](int ks, int nb, uint32_t (&bf)[4]) {
            const int row = ks * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
            if constexpr (L == 0) ldmatrix_x4_trans(bf, smem_u32(a + row * BS + nb * 16 + (lane >> 4) * 8));
            else ldmatrix_x4_trans(bf, smem_u32(a + blocked(row, nb * 2 + (lane >> 4), CIN)));
            if constexpr (L > 0) {
                using ActPrev = typename Spec::template Act<(L > 0 ? L - 1 : 0)>;
#pragma unroll
                for (int e = 0; e < 4; ++e)   // a register pairs two points of channel nb*16 + (e>>1)*8 + lane/4
                    bf[e] = h2_as_u32(act_forward2_same_channel<ActPrev>(u32_as_h2(bf[e]), nb * 16 + (e >> 1) * 8 + (lane >> 2)));
            }
        };
        // When the warps-across-blocks count is a multiple of the column blocks, all blocks of a warp share one column
        // block: its B fragment is loaded and activated once per k step instead of once per block (the activation is
        // the expensive part: config 4 puts a sine in front of a 64-wide layer)
        constexpr int NB = CIN / 16;
        constexpr bool SAME_NB = (WB % NB == 0);
#pragma unroll
        for (int ks = 0; ks < KSTEPS; ++ks) {
            if (ks % KW != wk) continue;
            uint32_t bf[4];
            if constexpr (SAME_NB) load_b(ks, wb % NB, bf);
#pragma unroll
            for (int b = 0; b < PB; ++b) {
                const int blk = wb + b * WB;
                if (blk >= NBLK) continue;
                const int mb = blk / NB, nb = blk % NB;
                // A fragment = delta^T (m = cout, k = point): transposing ldmatrix of the (point, cout) tile
                uint32_t af[4];
                ldmatrix_x4_trans(af, smem_u32(d + blocked(ks * 16 + (lane & 7) + ((lane >> 4) & 1) * 8, mb * 2 + ((lane >> 3) & 1), COUT)));
                if constexpr (!SAME_NB) load_b(ks, nb, bf);
                mma16816(acc[b][0], af, bf[0], bf[1]);
                mma16816(acc[b][1], af, bf[2], bf[3]);
                if constexpr (BIAS) {
                    if (nb == 0) mma16816(accB[b], af, 0x3C003C00u, 0x3C003C00u); // B = ones: row sums of delta^T
                }
            }
        }
        __syncthreads();
        buf = (buf + 1) % ST;
    }
    cp_async_wait<0>();

    // partial sums -> fp32 gradient vector (accumulated, callers zero it: reference semantics "+=",
    // kernels/network_weight_update_block.cuh:492)
    const int r = lane >> 2, q = lane & 3;
    float* gw = p.gradWeights + Spec::WOFF[L];
#pragma unroll
    for (int b = 0; b < PB; ++b) {
        const int blk = wb + b * WB;
        if (blk >= NBLK) continue;
        const int mb = blk / (CIN / 16), nb = blk % (CIN / 16);
#pragma unroll
        for (int h = 0; h < 2; ++h)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int m = mb * 16 + r + (e >> 1) * 8;
                const int n = nb * 16 + h * 8 + q * 2 + (e & 1);
                const float v = acc[b][h][e];
                if (v != 0.f) red_add_f32(gw + m * CIN + n, v);
            }
        if constexpr (BIAS) {
            if (nb == 0 && q == 0) {
                float* gb = p.gradWeights + (BIAS ? Spec::BOFF[L] : 0);
                if (accB[b][0] != 0.f) red_add_f32(gb + mb * 16 + r, accB[b][0]);
                if (accB[b][2] != 0.f) red_add_f32(gb + mb * 16 + r + 8, accB[b][2]);
            }
        }
    }
}

template <class Spec, int L>
__device__ __forceinline__ void wgrad_dispatch(const LaunchArgs& p, unsigned char* smem)
{
    if constexpr (L < Spec::NUM_LAYERS) {
        const int first = WgradSplit<Spec>::template begin<L>(gridDim.x), end = WgradSplit<Spec>::template begin<L + 1>(gridDim.x);
        if (static_cast<int>(blockIdx.x) < end) wgrad_layer<Spec, L>(p, smem, blockIdx.x - first, end - first);
        else wgrad_dispatch<Spec, L + 1>(p, smem);
    }
}

template <class Spec>
__global__ void __launch_bounds__(WG_WARPS * 32, 2)
wgrad_kernel(const __grid_constant__ LaunchArgs p)
{
    extern __shared__ __align__(16) unsigned char smem[];
    wgrad_dispatch<Spec, 0>(p, smem);
}

// ---- host-side launchers (compiled into each instantiation) -------------------------------------------------------
template <class Spec> struct TcLayout;     // fused_forward_tc.cuh
// Per-device latch for kernel attributes (a process may drive several GPUs): `run` performs `set` once per device and
// marks the device only after `set` succeeded, so a failed call is tried again and no launch can pass a latch whose
// attribute is not in place yet (a second thread that arrives early simply sets the same attribute again).
struct DeviceOnce {
    std::atomic<unsigned long long> done{0};
    template <class F>
    cudaError_t run(F set)
    {
        int d = 0;
        cudaError_t e = cudaGetDevice(&d);
        if (e != cudaSuccess) return e;
        const unsigned long long bit = 1ull << (d & 63);
        if ((done.load(std::memory_order_acquire) & bit) != 0) return cudaSuccess;
        e = set();
        if (e == cudaSuccess) done.fetch_or(bit, std::memory_order_release);
        return e;
    }
};

template <class Spec> struct TcLaunchers;
template <class Spec> struct PlaneLaunchers;
template <class Spec> struct SortLaunchers;

template <class Spec>
struct NetworkLaunchers {
    template <class K>
    static cudaError_t setSmem(K kernel, int bytes)
    {
        return cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
    }

    template <int MODE>
    static cudaError_t forward(const LaunchArgs& a, cudaStream_t s)
    {
        constexpr int smem = SmemLayout<Spec>::totalBytes();
        static DeviceOnce once;   // function attributes are per device
        auto k = fused_forward_kernel<Spec, MODE>;
        {
            const cudaError_t e = once.run([&] { return setSmem(k, smem); });
            if (e != cudaSuccess) return e;
        }
        int perSM = 0;
        cudaError_t e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&perSM, k, Spec::WARPS * 32, smem);
        if (e != cudaSuccess) return e;
        if (perSM < 1) perSM = 1;
        const long long tiles = (a.numel + TILE_POINTS - 1) / TILE_POINTS;
        long long blocks = (tiles + Spec::WARPS - 1) / Spec::WARPS;
        const long long cap = static_cast<long long>(a.numSMs) * perSM;
        if (blocks > cap) blocks = cap;
        if (blocks < 1) blocks = 1;
        k<<<static_cast<unsigned>(blocks), Spec::WARPS * 32, smem, s>>>(a);
        return cudaGetLastError();
    }

    template <int FLAGS>
    static cudaError_t backwardT(const LaunchArgs& a, cudaStream_t s)
    {
        constexpr int smem = SmemLayout<Spec>::totalBytes();
        static DeviceOnce once;   // function attributes are per device
        auto k = fused_backward_kernel<Spec, FLAGS>;
        {
            const cudaError_t e = once.run([&] { return setSmem(k, smem); });
            if (e != cudaSuccess) return e;
        }
        int perSM = 0;
        cudaError_t e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&perSM, k, Spec::WARPS * 32, smem);
        if (e != cudaSuccess) return e;
        if (perSM < 1) perSM = 1;
        const long long tiles = (a.numel + TILE_POINTS - 1) / TILE_POINTS;
        long long blocks = (tiles + Spec::WARPS - 1) / Spec::WARPS;
        const long long cap = static_cast<long long>(a.numSMs) * perSM;
        if (blocks > cap) blocks = cap;
        if (blocks < 1) blocks = 1;
        k<<<static_cast<unsigned>(blocks), Spec::WARPS * 32, smem, s>>>(a);
        return cudaGetLastError();
    }

    static cudaError_t backward(const LaunchArgs& a, cudaStream_t s)
    {
        if ((a.flags & FLAG_SPLIT_SCATTER) != 0) {
            if ((a.flags & 7) == 4) return backwardT<4 | FLAG_SPLIT_SCATTER>(a, s);
            if ((a.flags & 7) == 6) return backwardT<6 | FLAG_SPLIT_SCATTER>(a, s);
            return cudaErrorInvalidValue;
        }
        switch (a.flags & 7) {
        case 0: return cudaSuccess;
        case 1: return backwardT<1>(a, s);
        case 2: return backwardT<2>(a, s);
        case 3: return backwardT<3>(a, s);
        case 4: return backwardT<4>(a, s);
        case 5: return backwardT<5>(a, s);
        case 6: return backwardT<6>(a, s);
        default: return backwardT<7>(a, s);
        }
    }

    static cudaError_t wgrad(const LaunchArgs& a, cudaStream_t s)
    {
        constexpr int smem = WgradSmem<Spec>::bytes();
        static DeviceOnce once;   // function attributes are per device
        auto k = wgrad_kernel<Spec>;
        {
            const cudaError_t e = once.run([&] { return setSmem(k, smem); });
            if (e != cudaSuccess) return e;
        }
        // two CTAs per SM, fewer for small batches, never fewer than every layer needs to get one
        const long long slabs = (a.numel + WG_SLAB - 1) / WG_SLAB;
        long long ctas = static_cast<long long>(a.numSMs) * 2;
        if (ctas > slabs * Spec::NUM_LAYERS) ctas = slabs * Spec::NUM_LAYERS;
        if (ctas < WgradSplit<Spec>::minCtas()) ctas = WgradSplit<Spec>::minCtas();
        k<<<static_cast<unsigned>(ctas), WG_WARPS * 32, smem, s>>>(a);
        return cudaGetLastError();
    }

    static int launch(int kernel, const void* args, cudaStream_t s, int* launches)
    {
        const LaunchArgs& a = *static_cast<const LaunchArgs*>(args);
        cudaError_t e = cudaErrorInvalidValue;
        int n = 1;
        switch (kernel) {
        case KERNEL_INFERENCE:
            if constexpr (TcLayout<Spec>::eligible()) {
                // The tcgen05 kernel pays a fixed price per launch (tensor-memory allocation, operand staging for 148
                // large CTAs) and needs at least one 128-point tile per slot to use what it sets up; below that the
                // mma.sync kernel is quicker (config 1 at 2^16 points: 2.7 us against 4.7 us; config 2 at 2^16: 11.5
                // against 12.9 us, at 2^20: 89 against 62 us).
                const bool enough = a.numel >= TcLayout<Spec>::pointsPerCta() * a.numSMs;
                if (a.forcePath == 3 || (a.forcePath != 1 && enough)) { e = TcLaunchers<Spec>::inference(a, s); break; }
            }
            e = forward<0>(a, s);
            break;
        case KERNEL_ENCODE_PLANES:
            if constexpr (TcLayout<Spec>::eligible()) e = TcLaunchers<Spec>::encodePlanes(a, s);
            else e = cudaErrorNotSupported;   // the caller falls back to the fused gather
            break;
        case KERNEL_INFERENCE_PLANES:
            if constexpr (TcLayout<Spec>::eligible()) e = TcLaunchers<Spec>::inferencePlanes(a, s);
            else e = cudaErrorNotSupported;
            break;
        case KERNEL_FORWARD: e = forward<1>(a, s); break;
        case KERNEL_FORWARD_LOSS: e = forward<2>(a, s); break;
        case KERNEL_FORWARD_LOSS_PLANES:
            if constexpr (TcLayout<Spec>::eligible() && Spec::NUM_ENCODINGS > 0) e = forward<6>(a, s);
            else e = cudaErrorNotSupported;
            break;
        case KERNEL_BACKWARD: e = backward(a, s); n = (a.flags & 7) ? 1 : 0; break;
        case KERNEL_WGRAD: e = wgrad(a, s); break;
        case KERNEL_SCATTER_PLANES: e = PlaneLaunchers<Spec>::scatter(a, s); break;
        case KERNEL_SORT_POINTS: e = SortLaunchers<Spec>::sort(a, s, &n); break;
        case KERNEL_SCATTER_SORTED: e = SortLaunchers<Spec>::scatter(a, s); break;
        default: break;
        }
        if (launches) *launches = (e == cudaSuccess) ? n : 0;
        return static_cast<int>(e);
    }
};

} // namespace kernel
} // namespace qmlp
