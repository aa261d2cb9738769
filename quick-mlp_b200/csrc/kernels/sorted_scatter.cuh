// Spatially sorted training step: points in Morton-bin order, table gradients of the coarse levels summed in registers
// before they reach the L2.
//
// The table-gradient scatter (reference: one atomicAdd per corner and feature,
// src_cpp/include/qmlp/kernels/encoding_hashgrid.cuh:130-140) is bound by the rate at which the L2 executes reductions
// (one 32-byte sector per clock and slice, whatever the width), so the only way to make it faster is to send fewer of
// them. Points drawn at random share grid cells on every level whose cells are not much smaller than the spacing of the
// points (a batch of 2^20 points and a level of 54^3 cells: almost seven points per cell), but two such points sit in
// unrelated threads. So the step first sorts its points by a fine spatial bin (a counting sort: histogram, exclusive
// scan, reorder; the bins are cells of a regular grid over the bounding box, numbered in Morton order so that
// consecutive bins are neighbours in space). Every kernel after the sort reads the sorted copy, which also turns the
// coarse levels' gathers into L1 hits. In the scatter kernel a thread then walks a short run of consecutive sorted
// points on each coarse level and keeps the 2^D corner sums of the current cell in registers; they go to the table
// when the cell changes, one reduction per corner and run instead of one per corner and point. Finer levels go to the
// table directly, one point per thread, with corner pairs merged as in scatter_planes_kernel. (Sums of a whole brick of
// points in shared memory were measured first and dropped: shared-memory atomics run at about one lane per clock and
// SM, which made the coarse levels as slow as the reductions they replaced.)
//
// Measured on one B200, 3-D hash grid of 16 levels, 2^20 uniformly random points per step: gather 289 -> 227 us, scatter
// 538 -> 639 us (a quarter fewer reductions, but reductions of neighbouring points now reach the same L2 sectors at the
// same time and wait for each other; without the register sums 779 us), sort 140 us. The step is therefore only sorted on
// request; batches that arrive in spatial order (samples along rays) are the case it is kept for.
//
// Index arithmetic is the one of grid.cuh (bit-exact to the reference); only the order of the floating-point sums
// differs, as it does between any two runs of an atomic scatter.
#pragma once

namespace qmlp {
namespace kernel {

// first grid encoding of the network (its input channels and bounding box define the bins), -1: none
template <class Spec, int E = 0>
__host__ __device__ constexpr int first_plain_grid()
{
    if constexpr (E >= Spec::NUM_ENCODINGS) {
        return -1;
    } else {
        using Enc = typename Spec::template Enc<E>;
        if constexpr (Enc::IS_GRID) return E;
        else return first_plain_grid<Spec, E + 1>();
    }
}

template <int D>
__device__ __forceinline__ unsigned int morton_bin(const float (&pos)[D])
{
    constexpr int B = sort_bin_bits(D);
    unsigned int key = 0;
#pragma unroll
    for (int d = 0; d < D; ++d) {
        int c = static_cast<int>(pos[d] * static_cast<float>(1 << B));   // positions outside the box land in the border bins
        c = max(0, min((1 << B) - 1, c));
#pragma unroll
        for (int b = 0; b < B; ++b) key |= ((static_cast<unsigned int>(c) >> b) & 1u) << (b * D + d);
    }
    return key;
}

template <class Spec>
__global__ void __launch_bounds__(256) bin_count_kernel(const __grid_constant__ LaunchArgs p)
{
    constexpr int E = first_plain_grid<Spec>();
    using Enc = typename Spec::template Enc<(E < 0 ? 0 : E)>;
    const GridP& g = p.grids[Enc::SLOT];
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < p.numel;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
        RowReader in{p.input + i * p.inS0, p.inS1};
        float pos[Enc::D];
        grid_position<Enc::D, Enc::START>(g, in, pos);
        atomicAdd(p.binCounts + morton_bin<Enc::D>(pos), 1u);
    }
}

// exclusive prefix sum of the bin counts by one CTA: start[b] = first sorted point of bin b, start[NB] = all points;
// cursor[b] = start[b] is what the reorder kernel advances. Every warp scans a contiguous run of 32-bin chunks
// (coalesced loads, eight chunks requested ahead of their scans), then the 32 warp totals are scanned and added.
template <int NB>
__global__ void __launch_bounds__(1024) bin_scan_kernel(const unsigned int* __restrict__ counts, unsigned int* __restrict__ start,
                                                        unsigned int* __restrict__ cursor)
{
    static_assert(NB % 32 == 0, "whole chunks");
    constexpr int CHUNKS = NB / 32;
    constexpr int CPW = (CHUNKS + 31) / 32;   // chunks per warp
    constexpr int AHEAD = CPW < 8 ? CPW : 8;
    static_assert(CPW % AHEAD == 0, "whole batches");
    __shared__ unsigned int warpSums[32];
    const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
    unsigned int running = 0;
    // pass 1: exclusive sums relative to the warp's first bin, written to `start`
    for (int k0 = 0; k0 < CPW; k0 += AHEAD) {
        unsigned int v[AHEAD];
#pragma unroll
        for (int k = 0; k < AHEAD; ++k) {
            const int chunk = warp * CPW + k0 + k;
            v[k] = chunk < CHUNKS ? counts[chunk * 32 + lane] : 0u;
        }
#pragma unroll
        for (int k = 0; k < AHEAD; ++k) {
            unsigned int incl = v[k];
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const unsigned int u = __shfl_up_sync(0xffffffffu, incl, o);
                if (lane >= o) incl += u;
            }
            const int chunk = warp * CPW + k0 + k;
            if (chunk < CHUNKS) start[chunk * 32 + lane] = running + incl - v[k];
            running += __shfl_sync(0xffffffffu, incl, 31);
        }
    }
    if (lane == 0) warpSums[warp] = running;
    __syncthreads();
    if (warp == 0) {
        const unsigned int w = warpSums[lane];
        unsigned int wi = w;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const unsigned int u = __shfl_up_sync(0xffffffffu, wi, o);
            if (lane >= o) wi += u;
        }
        warpSums[lane] = wi - w;
        if (lane == 31) start[NB] = wi;
    }
    __syncthreads();
    // pass 2: add the warp's offset (the values were written by this same thread)
    const unsigned int base = warpSums[warp];
    for (int k0 = 0; k0 < CPW; k0 += AHEAD) {
        unsigned int v[AHEAD];
#pragma unroll
        for (int k = 0; k < AHEAD; ++k) {
            const int chunk = warp * CPW + k0 + k;
            v[k] = chunk < CHUNKS ? start[chunk * 32 + lane] : 0u;
        }
#pragma unroll
        for (int k = 0; k < AHEAD; ++k) {
            const int chunk = warp * CPW + k0 + k;
            if (chunk < CHUNKS) {
                start[chunk * 32 + lane] = base + v[k];
                cursor[chunk * 32 + lane] = base + v[k];
            }
        }
    }
}

template <class Spec>
__global__ void __launch_bounds__(256) bin_reorder_kernel(const __grid_constant__ LaunchArgs p)
{
    constexpr int E = first_plain_grid<Spec>();
    using Enc = typename Spec::template Enc<(E < 0 ? 0 : E)>;
    const GridP& g = p.grids[Enc::SLOT];
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < p.numel;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
        RowReader in{p.input + i * p.inS0, p.inS1};
        float x[Spec::NUM_INPUTS];
#pragma unroll
        for (int c = 0; c < Spec::NUM_INPUTS; ++c) x[c] = in(c);
        float pos[Enc::D];
#pragma unroll
        for (int k = 0; k < Enc::D; ++k) pos[k] = (x[k + Enc::START] - g.boxMin[k]) * g.boxInvSize[k];
        const unsigned int dst = atomicAdd(p.binCursor + morton_bin<Enc::D>(pos), 1u);
        float* xo = p.sortedInput + static_cast<long long>(dst) * Spec::NUM_INPUTS;
#pragma unroll
        for (int c = 0; c < Spec::NUM_INPUTS; ++c) xo[c] = x[c];
        if (p.sortedTarget != nullptr) {
#pragma unroll
            for (int c = 0; c < Spec::NUM_OUTPUTS; ++c)
                p.sortedTarget[static_cast<long long>(dst) * Spec::NUM_OUTPUTS + c] = __ldg(p.target + i * p.tS0 + c * p.tS1);
        }
    }
}

// ---- scatter of sorted points ------------------------------------------------------------------------------------------
constexpr int SORTED_THREADS = 128;
constexpr int SORTED_RUN = 8;                              // consecutive sorted points a thread walks on a coarse level
constexpr int SORTED_CHUNK = SORTED_THREADS * SORTED_RUN;  // points per CTA

template <int F>
__device__ __forceinline__ void read_adjoint_features(const __half* src, float (&adjF)[F])
{
    if constexpr (F == 2) {
        const float2 x = __half22float2(u32_as_h2(*reinterpret_cast<const uint32_t*>(src)));
        adjF[0] = x.x; adjF[1] = x.y;
    } else if constexpr (F == 4) {
        const uint2 u = *reinterpret_cast<const uint2*>(src);
        const float2 x = __half22float2(u32_as_h2(u.x)), y = __half22float2(u32_as_h2(u.y));
        adjF[0] = x.x; adjF[1] = x.y; adjF[2] = y.x; adjF[3] = y.y;
    } else {
#pragma unroll
        for (int i = 0; i < F; ++i) adjF[i] = __half2float(src[i]);
    }
}

// the 2^D corner sums of one cell -> gradient table; with two features per row, rows that are neighbours in memory go
// as one 16-byte reduction (same pairing rule as grid_level_scatter_paired)
template <int D, int F>
__device__ __forceinline__ void grid_scatter_cell(const GridP& g, const GridLevelP& lv, const GridCell<D>& c,
                                                  const float (&acc)[1 << D][F])
{
    const bool vec = g.vecOk != 0;
    if constexpr (F == 2) {
        if (vec) {
            const int pd = lv.hashed ? 0 : D - 1;
#pragma unroll
            for (int h = 0; h < (1 << (D - 1)); ++h) {
                const int b0 = pd == 0 ? (h << 1) : h;
                const int b1 = b0 | (1 << pd);
                const unsigned int eA = grid_corner_index<D, F>(g, c, lv, b0), eB = grid_corner_index<D, F>(g, c, lv, b1);
                // b0 / b1 depend on pd at run time: pick the sums with selects, not with dynamic indexing
                float a0 = 0.f, a1 = 0.f, c0 = 0.f, c1 = 0.f;
#pragma unroll
                for (int b = 0; b < (1 << D); ++b) {
                    if (b == b0) { a0 = acc[b][0]; a1 = acc[b][1]; }
                    if (b == b1) { c0 = acc[b][0]; c1 = acc[b][1]; }
                }
                float* pa = g.grad + eA;
                float* pb = g.grad + eB;
                if (eA == eB) {
                    red_add_v2_f32(pa, a0 + c0, a1 + c1);
                } else if (eB == eA + 2 && (reinterpret_cast<uintptr_t>(pa) & 15) == 0) {
                    red_add_v4_f32(pa, a0, a1, c0, c1);
                } else if (eA == eB + 2 && (reinterpret_cast<uintptr_t>(pb) & 15) == 0) {
                    red_add_v4_f32(pb, c0, c1, a0, a1);
                } else {
                    red_add_v2_f32(pa, a0, a1);
                    red_add_v2_f32(pb, c0, c1);
                }
            }
            return;
        }
    }
#pragma unroll
    for (int b = 0; b < (1 << D); ++b) grid_scatter_row<F>(g.grad, grid_corner_index<D, F>(g, c, lv, b), vec, 1.0f, acc[b]);
}

// One grid level of one encoding for the sorted points [base, end) of this CTA.
template <class Enc>
__device__ __forceinline__ void scatter_sorted_level(const LaunchArgs& p, const GridP& grid, int l, long long base, long long end)
{
    constexpr int D = Enc::D, F = Enc::F;
    const GridLevelP& lv = grid.levels[l];
    const int c0 = Enc::OUT_OFF + (Enc::CONCAT ? l * F : 0);
    const __half* plane = p.planes + p.planeStride * c0;

    // A level is walked in runs when the batch puts three or more points into two cells on average (the points are in
    // spatial order, so points of one cell follow each other); finer levels have nothing to sum.
    double cells = 1.0;
#pragma unroll
    for (int d = 0; d < D; ++d) cells *= static_cast<double>(lv.resolution - 1 > 0 ? lv.resolution - 1 : 1);
    const bool runs = p.runAggregation != 0 && static_cast<double>(p.numel) * 2.0 >= cells * 3.0;

    if (!runs) {
        for (long long pt = base + threadIdx.x; pt < end; pt += SORTED_THREADS) {
            RowReader in{p.input + pt * p.inS0, p.inS1};
            float adjF[F], pos[D];
            if (!scratch_ok(p, (plane - p.planes) + pt * F, F, p.planeHalfs, STATUS_PLANES)) continue;
            read_adjoint_features<F>(plane + pt * F, adjF);
            grid_position<D, Enc::START>(grid, in, pos);
            grid_level_scatter_paired<D, F>(grid, lv, pos, adjF);
        }
        return;
    }

    const long long first = base + static_cast<long long>(threadIdx.x) * SORTED_RUN;
    GridCell<D> cur;
    float acc[1 << D][F];
    bool open = false;
#pragma unroll 1
    for (int k = 0; k < SORTED_RUN; ++k) {
        const long long pt = first + k;
        if (pt >= end) break;
        RowReader in{p.input + pt * p.inS0, p.inS1};
        float adjF[F], pos[D];
        if (!scratch_ok(p, (plane - p.planes) + pt * F, F, p.planeHalfs, STATUS_PLANES)) continue;
        read_adjoint_features<F>(plane + pt * F, adjF);
        grid_position<D, Enc::START>(grid, in, pos);
        GridCell<D> c;
        grid_cell<D>(pos, lv.resolution, c);
        bool same = open;
#pragma unroll
        for (int d = 0; d < D; ++d) same = same && c.lo[d] == cur.lo[d] && c.hi[d] == cur.hi[d];
        if (!same) {
            if (open) grid_scatter_cell<D, F>(grid, lv, cur, acc);
#pragma unroll
            for (int d = 0; d < D; ++d) { cur.lo[d] = c.lo[d]; cur.hi[d] = c.hi[d]; }
#pragma unroll
            for (int b = 0; b < (1 << D); ++b)
#pragma unroll
                for (int i = 0; i < F; ++i) acc[b][i] = 0.f;
            open = true;
        }
#pragma unroll
        for (int b = 0; b < (1 << D); ++b) {
            const float w = grid_corner_weight<D>(c, b);
#pragma unroll
            for (int i = 0; i < F; ++i) acc[b][i] += w * adjF[i];
        }
    }
    if (open) grid_scatter_cell<D, F>(grid, lv, cur, acc);
}

template <class Spec, int E>
__device__ __forceinline__ void scatter_sorted_group(const LaunchArgs& p, int g, long long base, long long end)
{
    if constexpr (E < Spec::NUM_ENCODINGS) {
        using Enc = typename Spec::template Enc<E>;
        using SG = ScatterGroups<Spec, E>;
        if (g >= SG::before() + SG::own()) {
            scatter_sorted_group<Spec, E + 1>(p, g, base, end);
            return;
        }
        if constexpr (Enc::IS_GRID) {
            const GridP& grid = p.grids[Enc::SLOT];
            if (grid.grad == nullptr) return;
            scatter_sorted_level<Enc>(p, grid, g - SG::before(), base, end);
        }
    }
}

template <class Spec>
__global__ void __launch_bounds__(SORTED_THREADS, 6) scatter_sorted_kernel(const __grid_constant__ LaunchArgs p)
{
    constexpr int groups = scatter_group_count<Spec>();
    const long long base = static_cast<long long>(blockIdx.x) * SORTED_CHUNK;
    const long long end = base + SORTED_CHUNK < p.numel ? base + SORTED_CHUNK : p.numel;
    // the CTAs start at different levels, so that at any moment the reductions in flight spread over all tables
    const int first = static_cast<int>(blockIdx.x % groups);
    for (int gi = 0; gi < groups; ++gi) {
        int g = first + gi;
        if (g >= groups) g -= groups;
        scatter_sorted_group<Spec, 0>(p, g, base, end);
    }
}

template <class Spec>
struct SortLaunchers {
    static constexpr int E0 = first_plain_grid<Spec>();

    static constexpr int dims()
    {
        if constexpr (E0 < 0) return 1;
        else return Spec::template Enc<E0>::D;
    }

    // count, scan, reorder; `launches` receives the number of kernels
    static cudaError_t sort(const LaunchArgs& a, cudaStream_t s, int* launches)
    {
        if (launches) *launches = 0;
        if constexpr (E0 < 0) {
            return cudaErrorNotSupported;
        } else {
            constexpr int NB = sort_bin_count(dims());
            if (!a.binCounts || !a.binStart || !a.binCursor || !a.sortedInput) return cudaErrorInvalidValue;
            cudaError_t e = cudaMemsetAsync(a.binCounts, 0, sizeof(unsigned int) * NB, s);
            if (e != cudaSuccess) return e;
            // one point per thread (the loops only matter beyond 2^30 points): the reorder kernel waits for the value its
            // atomic returns, so what it reaches depends on how many of them are in flight
            long long bx = (a.numel + 255) / 256;
            const long long cap = 1ll << 22;
            if (bx > cap) bx = cap;
            if (bx < 1) bx = 1;
            bin_count_kernel<Spec><<<static_cast<unsigned>(bx), 256, 0, s>>>(a);
            bin_scan_kernel<NB><<<1, 1024, 0, s>>>(a.binCounts, a.binStart, a.binCursor);
            bin_reorder_kernel<Spec><<<static_cast<unsigned>(bx), 256, 0, s>>>(a);
            if (launches) *launches = 3;
            return cudaGetLastError();
        }
    }

    // `a.input` is the sorted copy
    static cudaError_t scatter(const LaunchArgs& a, cudaStream_t s)
    {
        constexpr int groups = scatter_group_count<Spec>();
        if constexpr (groups == 0 || E0 < 0) {
            return groups == 0 ? cudaSuccess : cudaErrorNotSupported;
        } else {
            long long bx = (a.numel + SORTED_CHUNK - 1) / SORTED_CHUNK;
            if (bx < 1) bx = 1;
            scatter_sorted_kernel<Spec><<<static_cast<unsigned>(bx), SORTED_THREADS, 0, s>>>(a);
            return cudaGetLastError();
        }
    }
};

} // namespace kernel
} // namespace qmlp
