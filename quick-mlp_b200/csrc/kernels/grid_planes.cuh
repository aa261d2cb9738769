// Level-major encoding pass for networks whose grid tables do not fit in L2.
//
// When the gather runs inside the fused kernel, every warp walks through all levels of its own points, so at any moment
// the SMs touch all tables at once: with tables far larger than the 126 MB L2 (a 4-D grid of 16 levels of which 12 are hashed
// tables of 2^22 rows) nearly every corner fetch is a random 32-byte DRAM sector. This pass reorders the work instead
// of the data: the encodings of a chunk of points are computed one level at a time by the whole GPU (blockIdx.y =
// level, the slow grid dimension), so the table of the level being processed (32 MB in fp16) stays resident in L2 and
// corner fetches hit it there. The features go to level-major planes ([level][point][F] halfs, coalesced 4/8/16-byte
// stores); the layer-chain kernel then reads its layer-0 operand from the planes (coalesced) instead of gathering.
// The chunk is sized so that planes and one table level together stay inside L2.
//
// Same arithmetic as the fused gather (grid.cuh; reference: src_cpp/include/qmlp/kernels/encoding_hashgrid.cuh:267-336).
#pragma once
#include "fused_network.cuh"

namespace qmlp {
namespace kernel {

// "groups": one per level of a concatenating grid, one for an adding grid, one for an identity encoding
template <class Spec, int E>
struct PlaneGroups {
    using Enc = typename Spec::template Enc<E>;
    __host__ __device__ static constexpr int own()
    {
        if constexpr (Enc::IS_GRID) return Enc::CONCAT ? Enc::L : 1;
        else return 1;
    }
    __host__ __device__ static constexpr int before()
    {
        if constexpr (E == 0) return 0;
        else return PlaneGroups<Spec, E - 1>::before() + PlaneGroups<Spec, E - 1>::own();
    }
};
template <class Spec>
__host__ __device__ constexpr int plane_group_count()
{
    return PlaneGroups<Spec, Spec::NUM_ENCODINGS - 1>::before() + PlaneGroups<Spec, Spec::NUM_ENCODINGS - 1>::own();
}

template <int W>
__device__ __forceinline__ void store_halfs(const LaunchArgs& p, __half* dst, const float (&v)[W])
{
    if (!scratch_ok(p, dst - p.planes, W, p.planeHalfs, STATUS_PLANES)) return;
    if constexpr (W == 2) {
        *reinterpret_cast<__half2*>(dst) = __floats2half2_rn(v[0], v[1]);
    } else if constexpr (W == 4) {
        uint2 u;
        u.x = h2_as_u32(__floats2half2_rn(v[0], v[1]));
        u.y = h2_as_u32(__floats2half2_rn(v[2], v[3]));
        *reinterpret_cast<uint2*>(dst) = u;
    } else if constexpr (W == 8) {
        uint4 u;
        u.x = h2_as_u32(__floats2half2_rn(v[0], v[1]));
        u.y = h2_as_u32(__floats2half2_rn(v[2], v[3]));
        u.z = h2_as_u32(__floats2half2_rn(v[4], v[5]));
        u.w = h2_as_u32(__floats2half2_rn(v[6], v[7]));
        *reinterpret_cast<uint4*>(dst) = u;
    } else {
#pragma unroll
        for (int i = 0; i < W; ++i) dst[i] = __float2half(v[i]);
    }
}

// features of group `g` (relative to all groups) for one point -> its plane
template <class Spec, int E>
__device__ __forceinline__ void encode_group(const LaunchArgs& p, int g, const RowReader& in, long long local)
{
    if constexpr (E < Spec::NUM_ENCODINGS) {
        using Enc = typename Spec::template Enc<E>;
        using PG = PlaneGroups<Spec, E>;
        if (g >= PG::before() + PG::own()) {
            encode_group<Spec, E + 1>(p, g, in, local);
            return;
        }
        if constexpr (!Enc::IS_GRID) {
            float v[Enc::N];
#pragma unroll
            for (int i = 0; i < Enc::N; ++i) v[i] = in(i + Enc::START);
            store_halfs<Enc::N>(p, p.planes + p.planeStride * Enc::OUT_OFF + local * Enc::N, v);
        } else {
            const GridP& grid = p.grids[Enc::SLOT];
            float pos[Enc::D];
            grid_position<Enc::D, Enc::START>(grid, in, pos);
            float feat[Enc::F];
            if constexpr (Enc::CONCAT) {
                const int l = g - PG::before();
                grid_level_forward<Enc::D, Enc::F, Enc::HALF_TABLE>(grid, grid.levels[l], pos, feat);
                store_halfs<Enc::F>(p, p.planes + p.planeStride * (Enc::OUT_OFF + l * Enc::F) + local * Enc::F, feat);
            } else {
#pragma unroll
                for (int i = 0; i < Enc::F; ++i) feat[i] = 0.f;
                for (int l = 0; l < Enc::L; ++l) {
                    float f[Enc::F];
                    grid_level_forward<Enc::D, Enc::F, Enc::HALF_TABLE>(grid, grid.levels[l], pos, f);
#pragma unroll
                    for (int i = 0; i < Enc::F; ++i) feat[i] += f[i];
                }
                store_halfs<Enc::F>(p, p.planes + p.planeStride * Enc::OUT_OFF + local * Enc::F, feat);
            }
        }
    }
}

// registers that hold one level's corner rows while its gathers are in flight; decides how many CTAs share an SM
template <class Spec, int E = 0>
__host__ __device__ constexpr int plane_row_registers()
{
    if constexpr (E >= Spec::NUM_ENCODINGS) {
        return 0;
    } else {
        using Enc = typename Spec::template Enc<E>;
        int own = 0;
        if constexpr (Enc::IS_GRID) own = (1 << Enc::D) * ((Enc::HALF_TABLE && Enc::F % 2 == 0) ? Enc::F / 2 : Enc::F);
        const int rest = plane_row_registers<Spec, E + 1>();
        return own > rest ? own : rest;
    }
}
template <class Spec>
__host__ __device__ constexpr int plane_min_blocks()
{
#ifdef QMLP_PLANE_MIN_BLOCKS
    return QMLP_PLANE_MIN_BLOCKS;
#else
    return plane_row_registers<Spec>() <= 32 ? 4 : (plane_row_registers<Spec>() <= 48 ? 3 : 2);
#endif
}

template <class Spec>
__global__ void __launch_bounds__(256, plane_min_blocks<Spec>()) encode_planes_kernel(const __grid_constant__ LaunchArgs p)
{
    const int g = blockIdx.y;
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < p.numel;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
        RowReader in{p.input + i * p.inS0, p.inS1};
        encode_group<Spec, 0>(p, g, in, i);
    }
}

// ---- level-major scatter of the table gradients --------------------------------------------------------------------
// Counterpart of the encoding pass for the backward direction: the backward kernel leaves the adjoint of every grid
// feature in the planes (write_adjoint_planes), and this kernel turns them into table gradients: light threads, many
// CTAs per SM, nothing but coalesced plane reads and reductions (the backward kernel itself runs 16 warps per SM at 128
// registers and alternates between MMA and scatter phases). A "group" is one level of one grid.
template <class Spec, int E>
struct ScatterGroups {
    using Enc = typename Spec::template Enc<E>;
    __host__ __device__ static constexpr int own()
    {
        if constexpr (Enc::IS_GRID) return Enc::L;
        else return 0;
    }
    __host__ __device__ static constexpr int before()
    {
        if constexpr (E == 0) return 0;
        else return ScatterGroups<Spec, E - 1>::before() + ScatterGroups<Spec, E - 1>::own();
    }
};
template <class Spec>
__host__ __device__ constexpr int scatter_group_count()
{
    return ScatterGroups<Spec, Spec::NUM_ENCODINGS - 1>::before() + ScatterGroups<Spec, Spec::NUM_ENCODINGS - 1>::own();
}

template <class Spec, int E>
__device__ __forceinline__ void scatter_group(const LaunchArgs& p, int g, const RowReader& in, long long point)
{
    if constexpr (E < Spec::NUM_ENCODINGS) {
        using Enc = typename Spec::template Enc<E>;
        using SG = ScatterGroups<Spec, E>;
        if (g >= SG::before() + SG::own()) {
            scatter_group<Spec, E + 1>(p, g, in, point);
            return;
        }
        if constexpr (Enc::IS_GRID) {
            const GridP& grid = p.grids[Enc::SLOT];
            if (grid.grad == nullptr) return;
            const int l = g - SG::before();
            const int c0 = Enc::OUT_OFF + (Enc::CONCAT ? l * Enc::F : 0);
            const __half* src = p.planes + p.planeStride * c0 + point * Enc::F;
            if (!scratch_ok(p, src - p.planes, Enc::F, p.planeHalfs, STATUS_PLANES)) return;
            float adjF[Enc::F];
            if constexpr (Enc::F == 2) {
                const float2 x = __half22float2(u32_as_h2(*reinterpret_cast<const uint32_t*>(src)));
                adjF[0] = x.x; adjF[1] = x.y;
            } else if constexpr (Enc::F == 4) {
                const uint2 u = *reinterpret_cast<const uint2*>(src);
                const float2 x = __half22float2(u32_as_h2(u.x)), y = __half22float2(u32_as_h2(u.y));
                adjF[0] = x.x; adjF[1] = x.y; adjF[2] = y.x; adjF[3] = y.y;
            } else {
#pragma unroll
                for (int i = 0; i < Enc::F; ++i) adjF[i] = __half2float(src[i]);
            }
            float pos[Enc::D];
            grid_position<Enc::D, Enc::START>(grid, in, pos);
            grid_level_scatter_paired<Enc::D, Enc::F>(grid, grid.levels[l], pos, adjF);
        }
    }
}

constexpr int SCATTER_THREADS = 128;

template <class Spec>
__global__ void __launch_bounds__(SCATTER_THREADS, 1024 / SCATTER_THREADS) scatter_planes_kernel(const __grid_constant__ LaunchArgs p)
{
    constexpr int groups = scatter_group_count<Spec>();
    const long long tiles = (p.numel + SCATTER_THREADS - 1) / SCATTER_THREADS;
    // levels of this launch (a data-parallel step scatters the levels in a few launches, so that the all-reduce of the
    // levels that are finished runs under the scatter of the next ones)
    const int begin = p.scatterLevelEnd > 0 ? p.scatterLevelBegin : 0;
    const int count = (p.scatterLevelEnd > 0 ? (p.scatterLevelEnd < groups ? p.scatterLevelEnd : groups) : groups) - begin;
    if (count <= 0) return;
    // A CTA takes its points through all levels, starting at a level that depends on the CTA: at any moment the CTAs of
    // the GPU are spread over all levels, so the reductions in flight go to many different rows and L2 slices (with all
    // CTAs on one small level, reductions to the same row queue up behind each other).
    const int first = static_cast<int>(blockIdx.x % count);
    for (long long t = blockIdx.x; t < tiles; t += gridDim.x) {
        const long long i = t * SCATTER_THREADS + threadIdx.x;
        if (i >= p.numel) continue;
        RowReader in{p.input + i * p.inS0, p.inS1};
        for (int gi = 0; gi < count; ++gi) {
            int g = first + gi;
            if (g >= count) g -= count;
            scatter_group<Spec, 0>(p, begin + g, in, i);
        }
    }
}

template <class Spec>
struct PlaneLaunchers {
    static cudaError_t scatter(const LaunchArgs& a, cudaStream_t s)
    {
        constexpr int groups = scatter_group_count<Spec>();
        if constexpr (groups == 0) {
            return cudaSuccess;
        } else {
            // one CTA per SCATTER_THREADS points: the hardware scheduler refills an SM as soon as a CTA retires, so the SMs drain
            // together at the end (with fewer, looping CTAs some took one tile more than others)
            long long bx = (a.numel + SCATTER_THREADS - 1) / SCATTER_THREADS;
            const long long cap = 1ll << 30;
            if (bx > cap) bx = cap;
            if (bx < 1) bx = 1;
            scatter_planes_kernel<Spec><<<static_cast<unsigned>(bx), SCATTER_THREADS, 0, s>>>(a);
            return cudaGetLastError();
        }
    }
};

} // namespace kernel
} // namespace qmlp

#include "sorted_scatter.cuh"
