// Multi-resolution dense / hashed grid: cell lookup, N-linear gather, gradient scatter, input gradient.
//
// Integer path (cell coordinates, dense and hashed row index) follows the reference bit for bit:
// src_cpp/include/qmlp/kernels/encoding_hashgrid.cuh:18-24 (primes), :36-46 (dense: last coordinate fastest; hash:
// xor of coordinate*prime in uint32), :71-84 (mod table size, times F, plus level offset), :277-284 (cell).
// What differs is the memory side: all F features of a corner move as one vector load / one vector reduction,
// tables may be fp16, and the level table arrives as a kernel parameter.
#pragma once
#include "launch_args.h"
#include "mma.cuh"

namespace qmlp {
namespace kernel {

__device__ __forceinline__ constexpr unsigned int hash_prime(int d)
{
    return d == 0 ? 1u : d == 1 ? 43857811u : d == 2 ? 83857661u : d == 3 ? 73856093u : d == 4 ? 19349663u : 834927u;
}

template <int D>
struct GridCell {
    unsigned int lo[D], hi[D]; // corner coordinates
    float f[D];                // fractions
};

// encoding_hashgrid.cuh:277-284
template <int D>
__device__ __forceinline__ void grid_cell(const float (&pos)[D], int resolution, GridCell<D>& c)
{
    const int rm1 = resolution - 1;
#pragma unroll
    for (int i = 0; i < D; ++i) {
        float p = pos[i] * (resolution - 1);
        int ip = static_cast<int>(p);
        int l = max(0, min(rm1, ip));
        int h = max(0, min(rm1, ip + 1));
        c.lo[i] = static_cast<unsigned int>(l);
        c.hi[i] = static_cast<unsigned int>(h);
        c.f[i] = p - static_cast<float>(l);
    }
}

// Element index (row*F + level offset) of the grid vertex with integer coordinates `v`.
template <int D, int F>
__device__ __forceinline__ unsigned int grid_vertex_index(const unsigned int (&v)[D], const GridLevelP& lv)
{
    unsigned int idx;
    if (lv.hashed) {
        idx = v[0] * hash_prime(0);
#pragma unroll
        for (int k = 1; k < D; ++k) idx = (v[k] * hash_prime(k)) ^ idx;
        idx = idx & (lv.hashGridSize - 1u); // == idx % hashGridSize: the table size is always 1 << log2_hashmap_size
    } else {
        idx = v[0];
#pragma unroll
        for (int k = 1; k < D; ++k) idx = v[k] + idx * static_cast<unsigned int>(lv.resolution);
    }
    return idx * F + lv.offset;
}

// Element index of corner `bits` of a cell (bit k set -> high corner in dimension k). Every table access of every kernel
// takes its index from here, so this is where a QMLP_BOUNDS_CHECK build tests it: a row that does not lie inside the
// table is reported through the status word and replaced by row 0 of the table, and the kernel carries on.
template <int D, int F>
__device__ __forceinline__ unsigned int grid_corner_index(const GridP& g, const GridCell<D>& c, const GridLevelP& lv, int bits)
{
    unsigned int v[D];
#pragma unroll
    for (int k = 0; k < D; ++k) v[k] = ((bits >> k) & 1) ? c.hi[k] : c.lo[k];
    const unsigned int e = grid_vertex_index<D, F>(v, lv);
    if constexpr (BOUNDS_CHECK) {
        if (static_cast<unsigned long long>(e) + F > g.tableCount) {
            if (g.status != nullptr) atomicOr(g.status, STATUS_TABLE_ROW);
            return 0u;
        }
    }
    return e;
}

// encoding_hashgrid.cuh:177-185,209-215: product taken from dimension D-1 down to 0
template <int D>
__device__ __forceinline__ float grid_corner_weight(const GridCell<D>& c, int bits)
{
    float w = 1.f;
#pragma unroll
    for (int k = D - 1; k >= 0; --k) w *= ((bits >> k) & 1) ? c.f[k] : (1.f - c.f[k]);
    return w;
}

template <int F, bool HALF>
__device__ __forceinline__ void grid_load_row(const void* table, unsigned int e, bool vec, float (&v)[F])
{
    if constexpr (HALF) {
        const __half* t = static_cast<const __half*>(table) + e;
        if constexpr (F == 2) {
            if (vec) { __half2 h = u32_as_h2(ldg_nc_u32(t)); float2 x = __half22float2(h); v[0] = x.x; v[1] = x.y; return; }
        } else if constexpr (F == 4) {
            if (vec) {
                uint2 u = ldg_nc_u64(t);
                float2 a = __half22float2(u32_as_h2(u.x)), b = __half22float2(u32_as_h2(u.y));
                v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y; return;
            }
        } else if constexpr (F == 8) {
            if (vec) {
                uint4 u = ldg_nc_u128(t);
                float2 a = __half22float2(u32_as_h2(u.x)), b = __half22float2(u32_as_h2(u.y));
                float2 c = __half22float2(u32_as_h2(u.z)), d = __half22float2(u32_as_h2(u.w));
                v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y; v[4] = c.x; v[5] = c.y; v[6] = d.x; v[7] = d.y; return;
            }
        }
#pragma unroll
        for (int i = 0; i < F; ++i) v[i] = __half2float(__ldg(t + i));
    } else {
        const float* t = static_cast<const float*>(table) + e;
        if constexpr (F == 2) {
            if (vec) { uint2 u = ldg_nc_u64(t); v[0] = __uint_as_float(u.x); v[1] = __uint_as_float(u.y); return; }
        } else if constexpr (F == 4) {
            if (vec) {
                uint4 u = ldg_nc_u128(t);
                v[0] = __uint_as_float(u.x); v[1] = __uint_as_float(u.y); v[2] = __uint_as_float(u.z); v[3] = __uint_as_float(u.w);
                return;
            }
        } else if constexpr (F == 8) {
            if (vec) {
                uint4 u = ldg_nc_u128(t), w = ldg_nc_u128(t + 4);
                v[0] = __uint_as_float(u.x); v[1] = __uint_as_float(u.y); v[2] = __uint_as_float(u.z); v[3] = __uint_as_float(u.w);
                v[4] = __uint_as_float(w.x); v[5] = __uint_as_float(w.y); v[6] = __uint_as_float(w.z); v[7] = __uint_as_float(w.w);
                return;
            }
        }
#pragma unroll
        for (int i = 0; i < F; ++i) v[i] = __ldg(t + i);
    }
}

template <int F>
__device__ __forceinline__ void grid_scatter_row(float* grad, unsigned int e, bool vec, float w, const float (&a)[F])
{
    float* g = grad + e;
    if constexpr (F == 2) {
        if (vec) { red_add_v2_f32(g, w * a[0], w * a[1]); return; }
    } else if constexpr (F % 4 == 0) {
        if (vec) {
#pragma unroll
            for (int i = 0; i < F; i += 4) red_add_v4_f32(g + i, w * a[i], w * a[i + 1], w * a[i + 2], w * a[i + 3]);
            return;
        }
    }
#pragma unroll
    for (int i = 0; i < F; ++i) red_add_f32(g + i, w * a[i]);
}

// position in the unit cube, encoding_hashgrid.cuh:316-320
template <int D, int START, class In>
__device__ __forceinline__ void grid_position(const GridP& g, const In& input, float (&pos)[D])
{
#pragma unroll
    for (int i = 0; i < D; ++i) pos[i] = (input(i + START) - g.boxMin[i]) * g.boxInvSize[i];
}

// Interpolated features of one level (fp32 blend), encoding_hashgrid.cuh:267-293.
template <int D, int F, bool HALF>
__device__ __forceinline__ void grid_level_forward(const GridP& g, const GridLevelP& lv, const float (&pos)[D], float (&feat)[F])
{
    GridCell<D> c;
    grid_cell<D>(pos, lv.resolution, c);
    const bool vec = g.vecOk != 0;
    if constexpr (HALF && (F == 2 || F == 4 || F == 8)) {
        // fp16 rows stay packed while the loads are in flight (half the registers of the unpacked rows, so more warps
        // fit on the SM to hide the gather latency); same blend order as below
        if (vec) {
            uint32_t raw[1 << D][F / 2];
#pragma unroll
            for (int b = 0; b < (1 << D); ++b) {
                const __half* t = static_cast<const __half*>(g.table) + grid_corner_index<D, F>(g, c, lv, b);
                if constexpr (F == 2) {
                    raw[b][0] = ldg_nc_u32(t);
                } else if constexpr (F == 4) {
                    const uint2 u = ldg_nc_u64(t);
                    raw[b][0] = u.x; raw[b][1] = u.y;
                } else {
                    const uint4 u = ldg_nc_u128(t);
                    raw[b][0] = u.x; raw[b][1] = u.y; raw[b][2] = u.z; raw[b][3] = u.w;
                }
            }
#pragma unroll
            for (int i = 0; i < F; ++i) feat[i] = 0.f;
#pragma unroll
            for (int b = 0; b < (1 << D); ++b) {
                const float w = grid_corner_weight<D>(c, b);
#pragma unroll
                for (int i = 0; i < F / 2; ++i) {
                    const float2 x = __half22float2(u32_as_h2(raw[b][i]));
                    feat[2 * i] += w * x.x;
                    feat[2 * i + 1] += w * x.y;
                }
            }
            return;
        }
    }
    float rows[1 << D][F];
    // issue every corner load before the blend so they are all in flight together
#pragma unroll
    for (int b = 0; b < (1 << D); ++b) grid_load_row<F, HALF>(g.table, grid_corner_index<D, F>(g, c, lv, b), vec, rows[b]);
#pragma unroll
    for (int i = 0; i < F; ++i) feat[i] = 0.f;
#pragma unroll
    for (int b = 0; b < (1 << D); ++b) {
        const float w = grid_corner_weight<D>(c, b);
#pragma unroll
        for (int i = 0; i < F; ++i) feat[i] += w * rows[b][i];
    }
}

// Adjoint of one level: scatter w*adjF to the corners (encoding_hashgrid.cuh:130-140) and, when requested,
// the gradient with respect to the unit-cube position. The position gradient carries the factor
// (resolution-1) of p = pos*(resolution-1), which the reference leaves out (encoding_hashgrid.cuh:224-239).
template <int D, int F, bool HALF, bool PARAM_GRAD, bool INPUT_GRAD>
__device__ __forceinline__ void grid_level_adjoint(const GridP& g, const GridLevelP& lv, const float (&pos)[D],
                                                   const float (&adjF)[F], float (&adjPos)[D])
{
    GridCell<D> c;
    grid_cell<D>(pos, lv.resolution, c);
    const bool vec = g.vecOk != 0;
    float lvl[D];
#pragma unroll
    for (int k = 0; k < D; ++k) lvl[k] = 0.f;
#pragma unroll
    for (int b = 0; b < (1 << D); ++b) {
        const unsigned int e = grid_corner_index<D, F>(g, c, lv, b);
        if constexpr (PARAM_GRAD) grid_scatter_row<F>(g.grad, e, vec, grid_corner_weight<D>(c, b), adjF);
        if constexpr (INPUT_GRAD) {
            float row[F];
            grid_load_row<F, HALF>(g.table, e, vec, row);
            float dot = 0.f;
#pragma unroll
            for (int i = 0; i < F; ++i) dot += adjF[i] * row[i];
#pragma unroll
            for (int k = 0; k < D; ++k) {
                float wk = 1.f;
#pragma unroll
                for (int j = D - 1; j >= 0; --j)
                    if (j != k) wk *= ((b >> j) & 1) ? c.f[j] : (1.f - c.f[j]);
                lvl[k] += (((b >> k) & 1) ? wk : -wk) * dot;
            }
        }
    }
    if constexpr (INPUT_GRAD) {
#pragma unroll
        for (int k = 0; k < D; ++k) adjPos[k] += lvl[k] * static_cast<float>(lv.resolution - 1);
    }
}

// Table gradient of one level with corner pairs merged (same sums as grid_level_adjoint<.., true, false>).
// The two corners that differ in the pairing dimension are neighbouring rows whenever the cell coordinate in that
// dimension is even: the hash multiplies dimension 0 by 1, so its low bit survives the xor (hashed levels: dimension
// 0); dense levels store the last coordinate fastest (dimension D-1). Two neighbouring rows of two fp32 features are
// one aligned 16-byte vector, i.e. one L2 reduction instead of two; at the upper border both corners are the same row
// and their weights are added first.
template <int D, int F>
__device__ __forceinline__ void grid_level_scatter_paired(const GridP& g, const GridLevelP& lv, const float (&pos)[D],
                                                          const float (&adjF)[F])
{
    GridCell<D> c;
    grid_cell<D>(pos, lv.resolution, c);
    const bool vec = g.vecOk != 0;
    if constexpr (F == 2) {
        if (vec) {
            const int pd = lv.hashed ? 0 : D - 1;
#pragma unroll
            for (int h = 0; h < (1 << (D - 1)); ++h) {
                const int b0 = pd == 0 ? (h << 1) : h;
                const int b1 = b0 | (1 << pd);
                const unsigned int eA = grid_corner_index<D, F>(g, c, lv, b0), eB = grid_corner_index<D, F>(g, c, lv, b1);
                const float wA = grid_corner_weight<D>(c, b0), wB = grid_corner_weight<D>(c, b1);
                float* pa = g.grad + eA;
                float* pb = g.grad + eB;
                if (eA == eB) {
                    red_add_v2_f32(pa, (wA + wB) * adjF[0], (wA + wB) * adjF[1]);
                } else if (eB == eA + 2 && (reinterpret_cast<uintptr_t>(pa) & 15) == 0) {
                    red_add_v4_f32(pa, wA * adjF[0], wA * adjF[1], wB * adjF[0], wB * adjF[1]);
                } else if (eA == eB + 2 && (reinterpret_cast<uintptr_t>(pb) & 15) == 0) {
                    red_add_v4_f32(pb, wB * adjF[0], wB * adjF[1], wA * adjF[0], wA * adjF[1]);
                } else {
                    red_add_v2_f32(pa, wA * adjF[0], wA * adjF[1]);
                    red_add_v2_f32(pb, wB * adjF[0], wB * adjF[1]);
                }
            }
            return;
        }
    }
#pragma unroll
    for (int b = 0; b < (1 << D); ++b)
        grid_scatter_row<F>(g.grad, grid_corner_index<D, F>(g, c, lv, b), vec, grid_corner_weight<D>(c, b), adjF);
}

} // namespace kernel
} // namespace qmlp
