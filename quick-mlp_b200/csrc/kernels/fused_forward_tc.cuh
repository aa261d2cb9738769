// Fused inference on the 5th-generation tensor cores (tcgen05.mma, accumulators in tensor memory).
//
// Same contract as fused_forward_kernel<Spec, 0> (replaces NetworkKernelInferenceAndForward,
// src_cpp/include/qmlp/kernels/network_forward.cuh:34-114, and Layer::inference, kernels/layer.cuh:101-181), different
// machine mapping:
//   * one persistent CTA per SM; all weight matrices are staged once in shared memory in the K-major, 128-byte
//     swizzled operand layout the tensor core reads through a shared-memory descriptor. The staging is done by the
//     tensor memory accelerator: one thread issues a tiled bulk copy (cp.async.bulk.tensor.2d, 128-byte swizzle) per
//     weight matrix and 64-wide K block through tensor maps the launcher encodes over the caller's parameter vector,
//     all onto one mbarrier; no cluster multicast, the source is this GPU's own memory;
//   * the CTA consists of 1, 2, 3, 4 or 8 warpgroups of 128 threads (as many as shared and tensor memory allow for
//     the spec's widths). A warpgroup owns one or two tile slots; a slot is one
//     tile of 128 points in flight: an activation operand buffer in shared memory plus an fp32 accumulator in tensor
//     memory. One thread = one point = one TMEM lane;
//   * per layer the warpgroup writes the rows of the A operand, synchronises on a named barrier, and one of its threads
//     issues K/16 MMAs D(128 x Cout) (+)= A(128 x 16) * W^T followed by tcgen05.commit onto the slot's mbarrier;
//   * the warpgroup waits on that mbarrier, reads its accumulator row with tcgen05.ld, rounds to half, adds the bias,
//     applies the activation and writes the row of the next layer's operand. With two slots it alternates between the
//     two tiles, so the MMAs of one run under the epilogue of the other; the warpgroups overlap each other anyway.
// Every mbarrier wait is bounded, and every stage ends in a warpgroup-wide vote: on a timeout the whole warpgroup leaves
// together, the CTA drains, tensor memory is released and the kernel reports through LaunchArgs::status.
#pragma once
#include <cuda.h>   // CUtensorMap and its enums; the encoder itself is fetched from the driver at run time
#include "fused_network.cuh"
#include "grid_planes.cuh"

namespace qmlp {
namespace kernel {

constexpr int TC_TILE = 128;            // points per tile = MMA M = TMEM lanes
constexpr uint32_t TC_SPIN_LIMIT = 1u << 24;

// ---- PTX wrappers ------------------------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ bool mbar_test(uint32_t bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
// bounded wait; false on timeout
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity)
{
    for (uint32_t i = 0; i < TC_SPIN_LIMIT; ++i)
        if (mbar_test(bar, parity)) return true;
    return false;
}
// barrier over the 128 threads of one warpgroup that also AND-reduces a predicate
__device__ __forceinline__ bool warpgroup_vote(int barrierId, bool pred)
{
    uint32_t r;
    asm volatile("{\n\t.reg .pred p, q;\n\tsetp.ne.b32 p, %2, 0;\n\tbar.red.and.pred q, %1, 128, p;\n\tselp.u32 %0, 1, 0, q;\n\t}"
                 : "=r"(r) : "r"(barrierId), "r"(static_cast<uint32_t>(pred)) : "memory");
    return r != 0;
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
// tiled bulk copy global -> shared of the box at (x, y) of a 2-D tensor map; completes on the mbarrier
__device__ __forceinline__ void tma_load_2d(uint32_t dstSmem, const void* tensorMap, int x, int y, uint32_t bar)
{
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(dstSmem), "l"(reinterpret_cast<uint64_t>(tensorMap)), "r"(x), "r"(y), "r"(bar) : "memory");
}
// stores through 32-bit shared-window addresses (one register per address instead of a generic pointer's two)
__device__ __forceinline__ void sts128(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d)
{
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}
__device__ __forceinline__ void sts32(uint32_t addr, uint32_t v) { asm volatile("st.shared.b32 [%0], %1;" ::"r"(addr), "r"(v) : "memory"); }
__device__ __forceinline__ void sts16(uint32_t addr, __half v)
{
    asm volatile("st.shared.b16 [%0], %1;" ::"r"(addr), "h"(__half_as_ushort(v)) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tmem_alloc(uint32_t smemDst, uint32_t cols)
{
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smemDst), "r"(cols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() { asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_dealloc(uint32_t addr, uint32_t cols)
{
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(addr), "r"(cols) : "memory");
}
__device__ __forceinline__ void umma_f16(uint32_t dTmem, uint64_t aDesc, uint64_t bDesc, uint32_t iDesc, uint32_t accumulate)
{
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                 ::"r"(dTmem), "l"(aDesc), "l"(bDesc), "r"(iDesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// 16 consecutive fp32 columns of this thread's TMEM lane
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, float (&v)[16])
{
    uint32_t r[16];
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                 : "r"(taddr) : "memory");
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}

// 64 consecutive fp32 columns of this thread's TMEM lane
__device__ __forceinline__ void tmem_ld64(uint32_t taddr, float (&v)[64])
{
    uint32_t r[64];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x64.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,"
        "%32,%33,%34,%35,%36,%37,%38,%39,%40,%41,%42,%43,%44,%45,%46,%47,%48,%49,%50,%51,%52,%53,%54,%55,%56,%57,%58,%59,%60,%61,%62,%63}, [%64];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
          "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]),
          "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]),
          "=r"(r[30]), "=r"(r[31]), "=r"(r[32]), "=r"(r[33]), "=r"(r[34]), "=r"(r[35]), "=r"(r[36]), "=r"(r[37]), "=r"(r[38]), "=r"(r[39]),
          "=r"(r[40]), "=r"(r[41]), "=r"(r[42]), "=r"(r[43]), "=r"(r[44]), "=r"(r[45]), "=r"(r[46]), "=r"(r[47]), "=r"(r[48]), "=r"(r[49]),
          "=r"(r[50]), "=r"(r[51]), "=r"(r[52]), "=r"(r[53]), "=r"(r[54]), "=r"(r[55]), "=r"(r[56]), "=r"(r[57]), "=r"(r[58]), "=r"(r[59]),
          "=r"(r[60]), "=r"(r[61]), "=r"(r[62]), "=r"(r[63])
        : "r"(taddr) : "memory");
#pragma unroll
    for (int i = 0; i < 64; ++i) v[i] = __uint_as_float(r[i]);
}

// Shared-memory matrix descriptor: K-major operand, 128-byte swizzle, 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t umma_desc_sw128(uint32_t smemAddr)
{
    return static_cast<uint64_t>((smemAddr >> 4) & 0x3FFFu)   // start address, 16-byte units
           | (1ull << 16)                                     // leading byte offset (unused for swizzled K-major)
           | (64ull << 32)                                    // stride byte offset: 1024 B between 8-row groups
           | (1ull << 46)                                     // descriptor version (sm_100)
           | (2ull << 61);                                    // layout type: SWIZZLE_128B
}
// Instruction descriptor: D fp32, A/B fp16, both K-major, shape M x N.
__host__ __device__ constexpr uint32_t umma_idesc_f16(int M, int N)
{
    return (1u << 4) | (static_cast<uint32_t>(N >> 3) << 17) | (static_cast<uint32_t>(M >> 4) << 24);
}

// byte offset of the 16-byte chunk `chunk` (8 halfs, counted along K) of row `row` inside an operand whose K extent is
// split in blocks of 64 halfs, each block ROWS x 128 bytes, chunk position xor-swizzled with the row (Swizzle<3,4,3>)
template <int ROWS>
__device__ __forceinline__ uint32_t sw128_offset(int row, int chunk)
{
    return static_cast<uint32_t>((chunk >> 3) * (ROWS * 128) + row * 128 + (((chunk & 7) ^ (row & 7)) << 4));
}

// ---- shared-memory plan ------------------------------------------------------------------------------------------------
template <class Spec>
struct TcLayout {
    static constexpr int NL = Spec::NUM_LAYERS;
    __host__ __device__ static constexpr int kBlocks(int l) { return (Spec::CIN[l] + 63) / 64; }
    __host__ __device__ static constexpr int wBytes(int l) { return kBlocks(l) * Spec::COUT[l] * 128; }
    __host__ __device__ static constexpr int wOffset(int l)
    {
        int o = 0;
        for (int i = 0; i < l; ++i) o += (wBytes(i) + 1023) / 1024 * 1024;
        return o;
    }
    __host__ __device__ static constexpr int weightBytes() { return wOffset(NL); }
    __host__ __device__ static constexpr int maxCin()
    {
        int m = 0;
        for (int i = 0; i < NL; ++i) m = Spec::CIN[i] > m ? Spec::CIN[i] : m;
        return m;
    }
    __host__ __device__ static constexpr int maxCout()
    {
        int m = 0;
        for (int i = 0; i < NL; ++i) m = Spec::COUT[i] > m ? Spec::COUT[i] : m;
        return m;
    }
    __host__ __device__ static constexpr int aBytes() { return (maxCin() + 63) / 64 * TC_TILE * 128; }
    // Bias operands. The bias is added by the tensor core: one extra K=16 MMA per biased layer whose A operand is a
    // constant block (every row = [1, 0, ..., 0], shared by all slots and layers) and whose B operand holds the bias in
    // its first K column. Both are K-major blocks of 16 halfs per row in the un-swizzled canonical layout
    // (8-row x 16-byte core matrices; see bias_block_offset).
    __host__ __device__ static constexpr int onesBytes() { return TC_TILE * 32; }
    __host__ __device__ static constexpr int biasOffset(int l)
    {
        int o = onesBytes();
        for (int i = 0; i < l; ++i) o += Spec::COUT[i] * 32;
        return o;
    }
    __host__ __device__ static constexpr int biasBytes() { return biasOffset(NL); }
    // accumulator columns per slot: power of two >= 32 so that SLOTS * cols is a legal allocation size
    __host__ __device__ static constexpr int accCols() { return maxCout() <= 32 ? 32 : maxCout() <= 64 ? 64 : maxCout() <= 128 ? 128 : 256; }
    __host__ __device__ static constexpr bool fits(int s) { return s * accCols() <= 512 && weightBytes() + s * aBytes() + biasBytes() + 4096 <= 220 * 1024; }
#ifndef QMLP_TC_MAX_WARPGROUPS
#define QMLP_TC_MAX_WARPGROUPS 8
#endif
    // 8 warpgroups (1024 threads, 64 registers each) with one slot each, or up to 4 warpgroups (128 registers) that
    // alternate between two slots when shared and tensor memory allow
    __host__ __device__ static constexpr int warpgroups() { return (QMLP_TC_MAX_WARPGROUPS >= 8 && fits(8)) ? 8 : fits(4) ? 4 : fits(3) ? 3 : fits(2) ? 2 : 1; }
    __host__ __device__ static constexpr int slotsPerWarpgroup() { return warpgroups() < 8 && fits(2 * warpgroups()) ? 2 : 1; }
    __host__ __device__ static constexpr int loadWidth() { return warpgroups() == 8 ? 32 : 64; }
    __host__ __device__ static constexpr int slots() { return warpgroups() * slotsPerWarpgroup(); }
    // points one CTA has in flight when every slot holds a tile
    __host__ __device__ static constexpr long long pointsPerCta() { return static_cast<long long>(TC_TILE) * slots(); }
    // tensor-memory allocation: a power of two >= 32 columns
    __host__ __device__ static constexpr int tmemCols()
    {
        int c = 32;
        while (c < slots() * accCols()) c *= 2;
        return c;
    }
    __host__ __device__ static constexpr bool eligible()
    {
        // (the plane kernels that come with this path know identity and grid encodings only)
        return maxCout() <= 128 && maxCin() <= 128 && fits(1) && !Spec::HAS_LINE;
    }
    __host__ __device__ static constexpr int aStart() { return weightBytes(); }
    __host__ __device__ static constexpr int biasStart() { return aStart() + slots() * aBytes(); }
    __host__ __device__ static constexpr int barStart() { return (biasStart() + biasBytes() + 127) / 128 * 128; }
    // 8 slot mbarriers of 8 bytes, the TMEM base word, the abort flag, the weight-staging mbarrier, 1 KB alignment slack
    __host__ __device__ static constexpr int totalBytes() { return barStart() + 8 * 8 + 64 + 1024; }
    // bytes the bulk copies of all weight matrices deliver (whole boxes: columns past Cin arrive as zeros)
    __host__ __device__ static constexpr int weightCopyBytes()
    {
        int b = 0;
        for (int i = 0; i < NL; ++i) b += wBytes(i);
        return b;
    }
};

// byte offset of element (row, k) of a K-major block of 16 halfs per row in the un-swizzled canonical layout:
// core matrices of 8 rows x 16 bytes (128 contiguous bytes); the two core matrices of a row group (k 0-7, k 8-15) are
// adjacent (leading byte offset 128), row groups are 256 bytes apart (stride byte offset 256)
__device__ __forceinline__ uint32_t bias_block_offset(int row, int k)
{
    return static_cast<uint32_t>((row >> 3) * 256 + (k >> 3) * 128 + (row & 7) * 16 + (k & 7) * 2);
}
__device__ __forceinline__ uint64_t umma_desc_k16_noswizzle(uint32_t smemAddr)
{
    return static_cast<uint64_t>((smemAddr >> 4) & 0x3FFFu)   // start address, 16-byte units
           | (8ull << 16)                                     // leading byte offset: 128 B between the two K halves
           | (16ull << 32)                                    // stride byte offset: 256 B between 8-row groups
           | (1ull << 46);                                    // descriptor version (sm_100); layout type 0 = no swizzle
}

// One tensor map per weight matrix: the (Cout, Cin) row-major fp16 block of the caller's parameter vector as a 2-D
// tensor, box = 64 halfs along K (one 128-byte swizzled row) x Cout rows.
template <class Spec>
struct TcWeightMaps {
    CUtensorMap m[Spec::NUM_LAYERS];
};

// issued by one thread: every weight matrix, K block by K block, into the operand layout (rows 128 bytes apart, the
// 16-byte chunks of a row xor-swizzled with the row index: exactly what sw128_offset describes)
template <class Spec, int L>
__device__ __forceinline__ void tc_issue_weight_copies(const TcWeightMaps<Spec>& maps, uint32_t sW, uint32_t bar)
{
    if constexpr (L < Spec::NUM_LAYERS) {
        using TL = TcLayout<Spec>;
        constexpr int COUT = Spec::COUT[L], KB = TL::kBlocks(L), OFF = TL::wOffset(L);
#pragma unroll
        for (int kb = 0; kb < KB; ++kb)
            tma_load_2d(sW + OFF + kb * COUT * 128, &maps.m[L], kb * 64, 0, bar);
        tc_issue_weight_copies<Spec, L + 1>(maps, sW, bar);
    }
}

// bias of layer L -> first K column of its block (whole CTA)
template <class Spec, int L>
__device__ __forceinline__ void tc_stage_bias(const LaunchArgs& p, unsigned char* sBias)
{
    if constexpr (L < Spec::NUM_LAYERS) {
        using TL = TcLayout<Spec>;
        constexpr int COUT = Spec::COUT[L];
        if constexpr (Spec::BOFF[L] >= 0) {
            unsigned char* bb = sBias + TL::biasOffset(L);
            for (int i = threadIdx.x; i < COUT * 16; i += blockDim.x) {
                const int r = i >> 4, k = i & 15;
                *reinterpret_cast<__half*>(bb + bias_block_offset(r, k)) = k == 0 ? p.weights[Spec::BOFF[L] + r] : __ushort_as_half(0);
            }
        }
        tc_stage_bias<Spec, L + 1>(p, sBias);
    }
}

// MMAs of layer L for one slot: K/16 instructions, then commit onto the slot's mbarrier (issued by one thread)
template <class Spec, int L>
// The descriptors differ from call to call only in the 14-bit start-address field (low word, 16-byte units), so the
// issuing thread keeps three base descriptors and adds compile-time offsets.
__device__ __forceinline__ void tc_issue_layer(uint32_t aSmem, uint32_t wSmem, uint32_t biasSmem, uint32_t dTmem, uint32_t fullBar)
{
    using TL = TcLayout<Spec>;
    const uint64_t aDesc0 = umma_desc_sw128(aSmem), wDesc0 = umma_desc_sw128(wSmem), biasDesc0 = umma_desc_k16_noswizzle(biasSmem);
    constexpr int CIN = Spec::CIN[L], COUT = Spec::COUT[L];
    constexpr uint32_t idesc = umma_idesc_f16(TC_TILE, COUT);
#pragma unroll
    for (int k = 0; k < CIN / 16; ++k) {
        const uint64_t aOff = static_cast<uint64_t>(((k >> 2) * (TC_TILE * 128) + (k & 3) * 32) >> 4);
        const uint64_t bOff = static_cast<uint64_t>((TL::wOffset(L) + (k >> 2) * (COUT * 128) + (k & 3) * 32) >> 4);
        umma_f16(dTmem, aDesc0 + aOff, wDesc0 + bOff, idesc, k > 0 ? 1u : 0u);
    }
    if constexpr (Spec::BOFF[L] >= 0)   // D += ones(128 x 16) * biasBlock(COUT x 16)^T : adds bias[n] to every row
        umma_f16(dTmem, biasDesc0, biasDesc0 + static_cast<uint64_t>(TL::biasOffset(L) >> 4), idesc, 1u);
    umma_commit(fullBar);
}

// ---- one warpgroup, one thread per point row -----------------------------------------------------------------------
struct TcSlot {                 // per-thread view of one tile slot
    uint32_t aRow;              // shared-window address of this thread's row of the slot's activation operand buffer
    uint32_t taddr;             // TMEM address of this thread's accumulator row
    uint32_t fullBar;           // mbarrier the MMAs of the slot commit to
    uint32_t fullParity;
    long long gRow;             // global point index of this thread in the slot's current tile
    bool active;                // the slot has a tile in this round
};

// byte offset of 16-byte chunk `chunk` inside a row of the operand whose row base (row * 128) is known: the K block's
// base plus the chunk position xor-swizzled with the row
__device__ __forceinline__ uint32_t sw128_row_offset(int row, int chunk)
{
    return static_cast<uint32_t>((chunk >> 3) * (TC_TILE * 128) + (((chunk & 7) ^ (row & 7)) << 4));
}

struct TcRowWriter {   // encoded features of one point -> swizzled row of the A operand
    uint32_t aRow;
    int row;
    __device__ __forceinline__ void operator()(int c, float v) const { sts16(aRow + sw128_row_offset(row, c >> 3) + (c & 7) * 2, __float2half(v)); }
    __device__ __forceinline__ void half(int c, __half v) const { sts16(aRow + sw128_row_offset(row, c >> 3) + (c & 7) * 2, v); }
    __device__ __forceinline__ void half2(int c, uint32_t v) const   // channels c, c + 1
    {
        if (c & 1) {
            half(c, __ushort_as_half(static_cast<unsigned short>(v & 0xffffu)));
            half(c + 1, __ushort_as_half(static_cast<unsigned short>(v >> 16)));
        } else {
            sts32(aRow + sw128_row_offset(row, c >> 3) + (c & 7) * 2, v);
        }
    }
};

// Stage 0: encode the point into the layer-0 operand. Stage L+1: epilogue of layer L. Each stage but the last ends
// by launching the MMAs of the next layer. Returns false, for the whole warpgroup at once, when a wait timed out.
template <class Spec, int ST, bool PLANES>
__device__ __forceinline__ bool tc_stage(const LaunchArgs& p, TcSlot& sl, uint32_t smemBase, int row, int barrierId, bool issuer)
{
    constexpr int NL = Spec::NUM_LAYERS;
    bool ok = true;
    if constexpr (ST == 0) {
        constexpr int CIN0 = Spec::CIN[0];
        // zero padding up to CIN0 and zero rows past the end of the batch
#pragma unroll
        for (int c = 0; c < CIN0 / 8; ++c) sts128(sl.aRow + sw128_row_offset(row, c), 0, 0, 0, 0);
        if (sl.gRow < p.numel) {
            if constexpr (PLANES) {
                read_planes_point<Spec, 0>(p, sl.gRow, TcRowWriter{sl.aRow, row});
            } else {
                RowReader in{p.input + sl.gRow * p.inS0, p.inS1};
                encode_point<Spec, 0>(p, in, TcRowWriter{sl.aRow, row});
            }
        }
    } else {
        constexpr int L = ST - 1;
        using Act = typename Spec::template Act<L>;
        constexpr int COUT = Spec::COUT[L];
        constexpr bool LAST = L == NL - 1;
        // tcgen05.ld is warp-collective: the decision to go on must be the same for all 32 lanes
        ok = __all_sync(0xffffffffu, mbar_wait(sl.fullBar, sl.fullParity));
        sl.fullParity ^= 1u;
        if (ok) {
            tc_fence_after();
            constexpr int NCOL = LAST ? (Spec::NUM_OUTPUTS + 15) / 16 * 16 : COUT;   // accumulator columns that are needed
            constexpr int LDW = TcLayout<Spec>::loadWidth();   // accumulator columns fetched per wait
            for (int c0 = 0; c0 < NCOL; c0 += LDW) {
                float v[LDW];   // bias already added by the tensor core
                if (LDW == 64 && NCOL - c0 >= 64) tmem_ld64(sl.taddr + c0, *reinterpret_cast<float (*)[64]>(&v[0]));
                else {
#pragma unroll
                    for (int g = 0; g < LDW / 16; ++g)
                        if (c0 + g * 16 < NCOL) tmem_ld16(sl.taddr + c0 + g * 16, *reinterpret_cast<float (*)[16]>(&v[g * 16]));
                }
                tmem_wait_ld();
#pragma unroll
                for (int g = 0; g < LDW / 16; ++g) {
                    if (c0 + g * 16 >= NCOL) continue;
                    uint32_t packed[8];
#pragma unroll
                    for (int i = 0; i < 8; ++i)
                        packed[i] = h2_as_u32(act_forward_f32x2<Act>(v[g * 16 + 2 * i], v[g * 16 + 2 * i + 1], c0 + g * 16 + 2 * i));
                    const int chunk = (c0 + g * 16) / 8;
                    if constexpr (!LAST) {
                        // row of the next layer's A operand: two 16-byte chunks
                        sts128(sl.aRow + sw128_row_offset(row, chunk), packed[0], packed[1], packed[2], packed[3]);
                        sts128(sl.aRow + sw128_row_offset(row, chunk + 1), packed[4], packed[5], packed[6], packed[7]);
                    } else if (sl.gRow < p.numel) {
                        // first NUM_OUTPUTS channels -> fp32 (kernels/network_forward.cuh:103-111)
#pragma unroll
                        for (int i = 0; i < 8; ++i) {
                            const float2 f = __half22float2(u32_as_h2(packed[i]));
                            const int c = c0 + g * 16 + 2 * i;
                            if (c < Spec::NUM_OUTPUTS) p.output[sl.gRow * p.outS0 + c * p.outS1] = f.x;
                            if (c + 1 < Spec::NUM_OUTPUTS) p.output[sl.gRow * p.outS0 + (c + 1) * p.outS1] = f.y;
                        }
                    }
                }
            }
        }
    }
    // All 128 rows of the operand are written and all accumulator reads are complete before the next MMAs start;
    // the same barrier carries the vote that makes a timeout a decision of the whole warpgroup.
    tc_fence_before();
    fence_proxy_async();    // generic-proxy writes of the operand become visible to the tensor core
    ok = warpgroup_vote(barrierId, ok);
    if constexpr (ST < NL) {
        if (ok && issuer) {
            // the issuing thread's row is the first of its warp: its addresses minus the row / lane parts are the slot's
            tc_fence_after();
            tc_issue_layer<Spec, ST>(sl.aRow - row * 128, smemBase, smemBase + TcLayout<Spec>::biasStart(),
                                     sl.taddr & 0x0000ffffu, sl.fullBar);
        }
    }
    return ok;
}

// all stages of up to SPW tiles, interleaved stage by stage
template <class Spec, int ST, int SPW, bool PLANES>
__device__ __forceinline__ bool tc_run_stages(const LaunchArgs& p, TcSlot (&sl)[SPW], uint32_t smemBase, int row, int barrierId, bool issuer)
{
    if constexpr (ST <= Spec::NUM_LAYERS) {
#pragma unroll
        for (int j = 0; j < SPW; ++j)
            if (sl[j].active) {   // uniform over the warpgroup
                if (!tc_stage<Spec, ST, PLANES>(p, sl[j], smemBase, row, barrierId, issuer)) return false;
            }
        return tc_run_stages<Spec, ST + 1, SPW, PLANES>(p, sl, smemBase, row, barrierId, issuer);
    } else {
        return true;
    }
}

template <class Spec, bool PLANES>
__global__ void __launch_bounds__(TcLayout<Spec>::warpgroups() * 128, 1)
fused_forward_tc_kernel(const __grid_constant__ LaunchArgs p, const __grid_constant__ TcWeightMaps<Spec> weightMaps)
{
    using TL = TcLayout<Spec>;
    constexpr int SLOTS = TL::slots();
    constexpr int SPW = TL::slotsPerWarpgroup();
    static_assert(SLOTS <= 8, "barrier area holds 8 slots");
    extern __shared__ unsigned char smemRaw[];
    // the swizzled operand layout needs 1024-byte alignment of every operand base
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smemRaw) + 1023) & ~static_cast<uintptr_t>(1023));
    unsigned char* sW = smem;
    unsigned char* sBias = smem + TL::biasStart();   // [ones block | bias block per layer]
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + TL::barStart());   // one per slot
    uint32_t* tmemSlot = reinterpret_cast<uint32_t*>(bars + 8);
    int* abortFlag = reinterpret_cast<int*>(tmemSlot + 1);
    uint64_t* weightBar = reinterpret_cast<uint64_t*>(tmemSlot + 4);

    const int warp = threadIdx.x >> 5;

    if (threadIdx.x == 0) {
        mbar_init(smem_u32(weightBar), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        mbar_expect_tx(smem_u32(weightBar), TL::weightCopyBytes());
        tc_issue_weight_copies<Spec, 0>(weightMaps, smem_u32(sW), smem_u32(weightBar));
    }
    tc_stage_bias<Spec, 0>(p, sBias);
    for (int i = threadIdx.x; i < TC_TILE * 16; i += blockDim.x)   // constant A operand of the bias MMA: every row = [1, 0, ..., 0]
        *reinterpret_cast<__half*>(sBias + bias_block_offset(i >> 4, i & 15)) = (i & 15) == 0 ? __ushort_as_half(0x3C00) : __ushort_as_half(0);
    if (threadIdx.x == 0) {
        *abortFlag = 0;
        for (int s = 0; s < SLOTS; ++s) mbar_init(smem_u32(bars + s), 1);   // one tcgen05.commit per phase
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        tmem_alloc(smem_u32(tmemSlot), TL::tmemCols());
        tmem_relinquish();
    }
    fence_proxy_async();   // bias blocks written by the threads -> visible to the tensor core
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmemBase = *tmemSlot;
    // the weights have arrived when the staging mbarrier completes its first phase (bounded wait like all others)
    const bool weightsIn = __all_sync(0xffffffffu, mbar_wait(smem_u32(weightBar), 0));

    // tile i of this CTA's sequence (global tile blockIdx.x + i * gridDim.x) goes to slot i % SLOTS
    // (32-bit tile counters: a launch holds fewer than 2^31 tiles of 128 points)
    const int numTiles = static_cast<int>((p.numel + TC_TILE - 1) / TC_TILE);
    const int firstTile = blockIdx.x;
    const int stride = gridDim.x;
    const int myTiles = firstTile < numTiles ? (numTiles - firstTile + stride - 1) / stride : 0;

    const int wg = warp >> 2;
    const int row = threadIdx.x & 127;                       // point row inside the tile = TMEM lane
    // the MMA-issuing thread of warpgroup wg sits in its warp (wg % 4), so the four issuers of a CTA run on four
    // different SM sub-partitions instead of all on the first one
    const bool issuer = row == (wg & 3) * 32;
    const uint32_t smemBase = smem_u32(smem);   // = the weight operands; everything else sits at fixed offsets from it
    TcSlot sl[SPW];
#pragma unroll
    for (int j = 0; j < SPW; ++j) {
        const int s = wg * SPW + j;
        sl[j].aRow = smemBase + TL::aStart() + s * TL::aBytes() + row * 128;
        sl[j].fullBar = smem_u32(bars + s);
        // (the allocation's lane field is 0, so the lane offset can be taken off again by masking)
        sl[j].taddr = tmemBase + s * TL::accCols() + (static_cast<uint32_t>((warp & 3) * 32) << 16);
        sl[j].fullParity = 0;
    }
    bool ok = weightsIn;
    for (int i = wg * SPW; i < myTiles && ok; i += SLOTS) {
#pragma unroll
        for (int j = 0; j < SPW; ++j) {
            sl[j].active = i + j < myTiles;
            sl[j].gRow = (firstTile + static_cast<long long>(i + j) * stride) * TC_TILE + row;
        }
        ok = tc_run_stages<Spec, 0, SPW, PLANES>(p, sl, smemBase, row, 1 + wg, issuer);
    }
    if (!ok) *abortFlag = 1;
    // drain: every warpgroup reaches this point (all waits are bounded), then tensor memory is released
    tc_fence_before();
    __syncthreads();
    if (warp == 0) {
        tc_fence_after();
        tmem_dealloc(tmemBase, TL::tmemCols());
    }
    if (threadIdx.x == 0 && *abortFlag && p.status != nullptr) atomicOr(p.status, STATUS_WAIT_TIMEOUT);
}

template <class Spec>
struct TcLaunchers {
    template <bool PLANES>
    static cudaError_t run(const LaunchArgs& a, cudaStream_t s)
    {
        using TL = TcLayout<Spec>;
        constexpr int smem = TL::totalBytes();
        constexpr int threads = TL::warpgroups() * 128;
        static DeviceOnce once;   // function attributes are per device
        auto k = fused_forward_tc_kernel<Spec, PLANES>;
        TcWeightMaps<Spec> maps;
        {
            const cudaError_t e = encodeWeightMaps(a.weights, maps);
            if (e != cudaSuccess) return e;
        }
        {
            const cudaError_t e = once.run([&] { return cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, smem); });
            if (e != cudaSuccess) return e;
        }
        const long long tiles = (a.numel + TC_TILE - 1) / TC_TILE;
        long long blocks = tiles < a.numSMs ? tiles : a.numSMs;
        if (blocks < 1) blocks = 1;
        k<<<static_cast<unsigned>(blocks), threads, smem, s>>>(a, maps);
        return cudaGetLastError();
    }
    // Tensor maps over the weight matrices of the bound parameter vector. Encoding is host arithmetic (no driver call
    // touches the device), a microsecond per matrix; the maps travel as a kernel parameter.
    static cudaError_t encodeWeightMaps(const __half* weights, TcWeightMaps<Spec>& maps)
    {
        using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                      const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                      CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
        static const EncodeFn encode = [] {
            void* fn = nullptr;
            cudaDriverEntryPointQueryResult found = cudaDriverEntryPointSymbolNotFound;
            if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &found) != cudaSuccess || found != cudaDriverEntryPointSuccess)
                fn = nullptr;
            return reinterpret_cast<EncodeFn>(fn);
        }();
        if (encode == nullptr) return cudaErrorNotSupported;
        if ((reinterpret_cast<uintptr_t>(weights) & 15u) != 0) return cudaErrorMisalignedAddress;
        for (int l = 0; l < Spec::NUM_LAYERS; ++l) {
            const cuuint64_t dims[2] = {static_cast<cuuint64_t>(Spec::CIN[l]), static_cast<cuuint64_t>(Spec::COUT[l])};
            const cuuint64_t strides[1] = {static_cast<cuuint64_t>(Spec::CIN[l]) * 2};   // bytes between rows
            const cuuint32_t box[2] = {64, static_cast<cuuint32_t>(Spec::COUT[l])};       // a narrower matrix is zero-filled up to 64
            const cuuint32_t elemStrides[2] = {1, 1};
            void* base = const_cast<__half*>(weights + Spec::WOFF[l]);
            if (encode(&maps.m[l], CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, base, dims, strides, box, elemStrides, CU_TENSOR_MAP_INTERLEAVE_NONE,
                       CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
                return cudaErrorInvalidValue;
        }
        return cudaSuccess;
    }
    static cudaError_t inference(const LaunchArgs& a, cudaStream_t s) { return run<false>(a, s); }
    static cudaError_t inferencePlanes(const LaunchArgs& a, cudaStream_t s) { return run<true>(a, s); }
    // level-major encoding pass: blockIdx.y = level (slow), blockIdx.x strides over the points of the chunk
    static cudaError_t encodePlanes(const LaunchArgs& a, cudaStream_t s)
    {
        constexpr int groups = plane_group_count<Spec>();
        long long bx = (a.numel + 255) / 256;
        const long long cap = static_cast<long long>(a.numSMs) * 8;
        if (bx > cap) bx = cap;
        if (bx < 1) bx = 1;
        encode_planes_kernel<Spec><<<dim3(static_cast<unsigned>(bx), groups), 256, 0, s>>>(a);
        return cudaGetLastError();
    }
};

} // namespace kernel
} // namespace qmlp
