// Fused inference on the 5th-generation tensor cores (tcgen05.mma, accumulators in tensor memory).
//
// Same contract as fused_forward_kernel<Spec, 0> (replaces NetworkKernelInferenceAndForward,
// src_cpp/include/qmlp/kernels/network_forward.cuh:34-114, and Layer::inference, kernels/layer.cuh:101-181), different
// machine mapping:
//   * one persistent CTA per SM; all weight matrices are staged once in shared memory in the K-major, 128-byte
//     swizzled operand layout the tensor core reads through a shared-memory descriptor;
//   * SLOTS point tiles of 128 points are in flight per CTA. Each slot owns one warpgroup (128 threads, one thread per
//     point = one TMEM lane), one activation operand buffer in shared memory, and one fp32 accumulator in tensor memory;
//   * one extra warp issues the MMAs: for slot s and layer l, K/16 instructions D(128 x Cout) (+)= A(128 x 16) * W^T,
//     then tcgen05.commit signals the slot's "accumulator full" mbarrier;
//   * the slot's warpgroup waits for that barrier, reads its accumulator row with tcgen05.ld, rounds to half, adds the
//     bias, applies the activation, writes the row of the next layer's A operand (swizzled) and signals "operand ready".
//     The epilogue of one slot overlaps the MMAs and epilogues of the others.
// Every wait is bounded: on a timeout the CTA raises an abort flag, all loops drain, tensor memory is released and the
// kernel reports through LaunchArgs::status instead of hanging.
#pragma once
#include "fused_network.cuh"

namespace qmlp {
namespace kernel {

constexpr int TC_TILE = 128;            // points per tile = MMA M = TMEM lanes
constexpr uint32_t TC_SPIN_LIMIT = 1u << 24;

// ---- PTX wrappers ------------------------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar)
{
    asm volatile("{\n\t.reg .b64 st;\n\tmbarrier.arrive.shared::cta.b64 st, [%0];\n\t}" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_test(uint32_t bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
// bounded wait; returns false (and raises the abort flag) on timeout or when another thread aborted
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abortFlag)
{
    for (uint32_t i = 0; i < TC_SPIN_LIMIT; ++i) {
        if (mbar_test(bar, parity)) return true;
        if ((i & 1023u) == 1023u && *abortFlag) return false;
    }
    *abortFlag = 1;
    return false;
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
    __host__ __device__ static constexpr int biasHalfs()
    {
        int o = 0;
        for (int i = 0; i < NL; ++i) o += Spec::COUT[i];
        return o;
    }
    __host__ __device__ static constexpr int biasOffset(int l)
    {
        int o = 0;
        for (int i = 0; i < l; ++i) o += Spec::COUT[i];
        return o;
    }
    // accumulator columns per slot: power of two >= 32 so that SLOTS * cols is a legal allocation size
    __host__ __device__ static constexpr int accCols() { return maxCout() <= 32 ? 32 : maxCout() <= 64 ? 64 : maxCout() <= 128 ? 128 : 256; }
    __host__ __device__ static constexpr int slots()
    {
        int s = 4;
        while (s > 1 && (s * accCols() > 512 || weightBytes() + s * aBytes() + 4096 > 220 * 1024)) s >>= 1;
        return s;
    }
    __host__ __device__ static constexpr bool eligible()
    {
        return maxCout() <= 128 && maxCin() <= 128 && weightBytes() + aBytes() + 4096 <= 220 * 1024;
    }
    __host__ __device__ static constexpr int aStart() { return weightBytes(); }
    __host__ __device__ static constexpr int biasStart() { return aStart() + slots() * aBytes(); }
    __host__ __device__ static constexpr int barStart() { return (biasStart() + biasHalfs() * 2 + 15) / 16 * 16; }
    // 16 mbarriers (8 "full" + 8 "ready" slots) of 8 bytes, the TMEM base word and the abort flag, 1 KB alignment slack
    __host__ __device__ static constexpr int totalBytes() { return barStart() + 16 * 8 + 64 + 1024; }
};

// weights of layer L -> swizzled K-major operand in shared memory (whole CTA)
template <class Spec, int L>
__device__ __forceinline__ void tc_stage_weights(const LaunchArgs& p, unsigned char* sW, __half* sBias)
{
    if constexpr (L < Spec::NUM_LAYERS) {
        using TL = TcLayout<Spec>;
        constexpr int CIN = Spec::CIN[L], COUT = Spec::COUT[L];
        constexpr int CH = CIN / 8;
        const __half* gW = p.weights + Spec::WOFF[L];
        unsigned char* dst = sW + TL::wOffset(L);
        for (int i = threadIdx.x; i < COUT * CH; i += blockDim.x) {
            const int r = i / CH, c = i % CH;
            *reinterpret_cast<uint4*>(dst + sw128_offset<COUT>(r, c)) = *reinterpret_cast<const uint4*>(gW + r * CIN + c * 8);
        }
        for (int i = threadIdx.x; i < COUT; i += blockDim.x)
            sBias[TL::biasOffset(L) + i] = Spec::BOFF[L] >= 0 ? p.weights[(Spec::BOFF[L] >= 0 ? Spec::BOFF[L] : 0) + i] : __ushort_as_half(0);
        tc_stage_weights<Spec, L + 1>(p, sW, sBias);
    }
}

// MMA issue for one (slot, layer): K/16 instructions, then commit to the slot's "full" barrier (one thread)
template <class Spec, int L>
__device__ __forceinline__ void tc_issue_layer(int layer, uint32_t aBase, uint32_t wBase, uint32_t dTmem, uint32_t fullBar)
{
    if constexpr (L < Spec::NUM_LAYERS) {
        if (layer == L) {
            using TL = TcLayout<Spec>;
            constexpr int CIN = Spec::CIN[L], COUT = Spec::COUT[L];
            constexpr uint32_t idesc = umma_idesc_f16(TC_TILE, COUT);
#pragma unroll
            for (int k = 0; k < CIN / 16; ++k) {
                const uint32_t aAddr = aBase + (k >> 2) * (TC_TILE * 128) + (k & 3) * 32;
                const uint32_t bAddr = wBase + TL::wOffset(L) + (k >> 2) * (COUT * 128) + (k & 3) * 32;
                umma_f16(dTmem, umma_desc_sw128(aAddr), umma_desc_sw128(bAddr), idesc, k > 0 ? 1u : 0u);
            }
            umma_commit(fullBar);
        } else {
            tc_issue_layer<Spec, L + 1>(layer, aBase, wBase, dTmem, fullBar);
        }
    }
}

// epilogue of layer L for one point row; returns false on abort
template <class Spec, int L>
__device__ __forceinline__ bool tc_epilogue_layers(const LaunchArgs& p, unsigned char* aBuf, const __half* sBias,
                                                   uint32_t taddr, uint32_t fullBar, uint32_t readyBar, uint32_t& fullParity,
                                                   int row, long long gRow, volatile int* abortFlag)
{
    using TL = TcLayout<Spec>;
    using Act = typename Spec::template Act<L>;
    constexpr int COUT = Spec::COUT[L];
    constexpr bool LAST = L == Spec::NUM_LAYERS - 1;
    constexpr bool BIAS = Spec::BOFF[L] >= 0;
    // tcgen05.ld is warp-collective: the decision to go on must be the same for all 32 lanes
    if (!__all_sync(0xffffffffu, mbar_wait(fullBar, fullParity, abortFlag))) return false;
    fullParity ^= 1u;
    tc_fence_after();
    const __half* bias = sBias + TL::biasOffset(L);
    constexpr int NCH = LAST ? (Spec::NUM_OUTPUTS + 15) / 16 : COUT / 16;   // 16-column groups that are needed
#pragma unroll
    for (int g0 = 0; g0 < NCH; g0 += 4) {
      // up to 64 accumulator columns in flight, one wait
      float vv[4][16];
#pragma unroll
      for (int gg = 0; gg < 4; ++gg)
          if (g0 + gg < NCH) tmem_ld16(taddr + (g0 + gg) * 16, vv[gg]);
      tmem_wait_ld();
#pragma unroll
      for (int gg = 0; gg < 4; ++gg) {
        const int g = g0 + gg;
        if (g >= NCH) continue;
        float (&v)[16] = vv[gg];
        uint32_t packed[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            __half2 h = __floats2half2_rn(v[2 * i], v[2 * i + 1]);
            if constexpr (BIAS) h = __hadd2(h, *reinterpret_cast<const __half2*>(bias + g * 16 + 2 * i));
            h = Act::forward2(h);
            packed[i] = h2_as_u32(h);
        }
        if constexpr (!LAST) {
            // row of the next layer's A operand: two 16-byte chunks
            *reinterpret_cast<uint4*>(aBuf + sw128_offset<TC_TILE>(row, 2 * g)) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
            *reinterpret_cast<uint4*>(aBuf + sw128_offset<TC_TILE>(row, 2 * g + 1)) = make_uint4(packed[4], packed[5], packed[6], packed[7]);
        } else {
            if (gRow < p.numel) {
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const float2 f = __half22float2(u32_as_h2(packed[i]));
                    const int c = g * 16 + 2 * i;
                    if (c < Spec::NUM_OUTPUTS) p.output[gRow * p.outS0 + c * p.outS1] = f.x;
                    if (c + 1 < Spec::NUM_OUTPUTS) p.output[gRow * p.outS0 + (c + 1) * p.outS1] = f.y;
                }
            }
        }
      }
    }
    if constexpr (!LAST) {
        tc_fence_before();      // the accumulator reads are complete before the next MMA may overwrite it
        fence_proxy_async();    // generic-proxy writes of the operand become visible to the tensor core
        mbar_arrive(readyBar);
        return tc_epilogue_layers<Spec, L + 1>(p, aBuf, sBias, taddr, fullBar, readyBar, fullParity, row, gRow, abortFlag);
    } else {
        tc_fence_before();
        return true;
    }
}

struct TcRowWriter {   // encoded features of one point -> swizzled row of the A operand
    unsigned char* aBuf;
    int row;
    __device__ __forceinline__ void operator()(int c, float v) const
    {
        *reinterpret_cast<__half*>(aBuf + sw128_offset<TC_TILE>(row, c >> 3) + (c & 7) * 2) = __float2half(v);
    }
};

template <class Spec>
__global__ void __launch_bounds__(TcLayout<Spec>::slots() * 128 + 32, 1)
fused_forward_tc_kernel(const __grid_constant__ LaunchArgs p)
{
    using TL = TcLayout<Spec>;
    constexpr int SLOTS = TL::slots();
    constexpr int NL = Spec::NUM_LAYERS;
    extern __shared__ unsigned char smemRaw[];
    // the swizzled operand layout needs 1024-byte alignment of every operand base
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smemRaw) + 1023) & ~static_cast<uintptr_t>(1023));
    unsigned char* sW = smem;
    unsigned char* sA = smem + TL::aStart();
    __half* sBias = reinterpret_cast<__half*>(smem + TL::biasStart());
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + TL::barStart());   // [SLOTS] full, [SLOTS] ready
    uint32_t* tmemSlot = reinterpret_cast<uint32_t*>(bars + 16);
    volatile int* abortFlag = reinterpret_cast<volatile int*>(tmemSlot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    constexpr int MMA_WARP = SLOTS * 4;

    tc_stage_weights<Spec, 0>(p, sW, sBias);
    if (threadIdx.x == 0) {
        *abortFlag = 0;
        for (int s = 0; s < SLOTS; ++s) {
            mbar_init(smem_u32(bars + s), 1);            // full: one tcgen05.commit
            mbar_init(smem_u32(bars + 8 + s), 128);      // ready: every thread of the warpgroup
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == MMA_WARP) {
        tmem_alloc(smem_u32(tmemSlot), SLOTS * TL::accCols());
        tmem_relinquish();
    }
    fence_proxy_async();   // staged weights -> visible to the tensor core
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmemBase = *tmemSlot;

    const long long numTiles = (p.numel + TC_TILE - 1) / TC_TILE;
    // tile t of this CTA's sequence goes to slot t % SLOTS
    const long long firstTile = blockIdx.x;
    const long long stride = gridDim.x;
    long long myTiles = firstTile < numTiles ? (numTiles - firstTile + stride - 1) / stride : 0;

    if (warp < MMA_WARP) {
        // ---------------- epilogue warpgroup of slot s ----------------
        const int s = warp >> 2;
        const int row = threadIdx.x & 127;                       // point row inside the tile = TMEM lane
        unsigned char* aBuf = sA + s * TL::aBytes();
        const uint32_t fullBar = smem_u32(bars + s), readyBar = smem_u32(bars + 8 + s);
        const uint32_t taddr = tmemBase + (static_cast<uint32_t>((warp & 3) * 32) << 16) + s * TL::accCols();
        uint32_t fullParity = 0;
        bool ok = true;
        for (long long i = s; i < myTiles && ok; i += SLOTS) {
            const long long tile = firstTile + i * stride;
            const long long gRow = tile * TC_TILE + row;
            // layer-0 operand: encodings of this thread's point (zero padding up to CIN0, zero rows past the end)
            constexpr int CIN0 = Spec::CIN[0];
#pragma unroll
            for (int c = 0; c < CIN0 / 8; ++c) *reinterpret_cast<uint4*>(aBuf + sw128_offset<TC_TILE>(row, c)) = make_uint4(0, 0, 0, 0);
            if (gRow < p.numel) {
                RowReader in{p.input + gRow * p.inS0, p.inS1};
                encode_point<Spec, 0>(p, in, TcRowWriter{aBuf, row});
            }
            tc_fence_before();
            fence_proxy_async();
            mbar_arrive(readyBar);
            ok = tc_epilogue_layers<Spec, 0>(p, aBuf, sBias, taddr, fullBar, readyBar, fullParity, row, gRow, abortFlag);
        }
    } else if (lane == 0) {
        // ---------------- MMA issue thread ----------------
        const uint32_t aBase = smem_u32(sA), wBase = smem_u32(sW);
        int layer[SLOTS];
        long long done[SLOTS];          // tiles finished per slot
        uint32_t readyParity[SLOTS];
        long long total = 0;
#pragma unroll
        for (int s = 0; s < SLOTS; ++s) {
            layer[s] = 0; done[s] = 0; readyParity[s] = 0;
        }
        long long perSlot[SLOTS];
#pragma unroll
        for (int s = 0; s < SLOTS; ++s) { perSlot[s] = myTiles > s ? (myTiles - s + SLOTS - 1) / SLOTS : 0; total += perSlot[s] * NL; }
        long long issued = 0;
        uint32_t idle = 0;
        while (issued < total) {
            bool any = false;
#pragma unroll
            for (int s = 0; s < SLOTS; ++s) {
                if (done[s] >= perSlot[s]) continue;
                if (!mbar_test(smem_u32(bars + 8 + s), readyParity[s])) continue;
                readyParity[s] ^= 1u;
                tc_fence_after();
                tc_issue_layer<Spec, 0>(layer[s], aBase + s * TL::aBytes(), wBase, tmemBase + s * TL::accCols(), smem_u32(bars + s));
                ++issued;
                any = true;
                if (++layer[s] == NL) { layer[s] = 0; ++done[s]; }
            }
            if (any) { idle = 0; continue; }
            if (++idle > TC_SPIN_LIMIT) { *abortFlag = 1; break; }
            if ((idle & 1023u) == 1023u && *abortFlag) break;
        }
    }
    // drain: every role reaches this point (all waits are bounded), then tensor memory is released
    tc_fence_before();
    __syncthreads();
    if (warp == MMA_WARP) {
        tc_fence_after();
        tmem_dealloc(tmemBase, SLOTS * TL::accCols());
    }
    if (threadIdx.x == 0 && *abortFlag && p.status != nullptr) atomicExch(p.status, 1);
}

template <class Spec>
struct TcLaunchers {
    static cudaError_t inference(const LaunchArgs& a, cudaStream_t s)
    {
        using TL = TcLayout<Spec>;
        constexpr int smem = TL::totalBytes();
        constexpr int threads = TL::slots() * 128 + 32;
        static bool configured = false;
        auto k = fused_forward_tc_kernel<Spec>;
        if (!configured) {
            cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
            if (e != cudaSuccess) return e;
            configured = true;
        }
        const long long tiles = (a.numel + TC_TILE - 1) / TC_TILE;
        long long blocks = tiles < a.numSMs ? tiles : a.numSMs;
        if (blocks < 1) blocks = 1;
        k<<<static_cast<unsigned>(blocks), threads, smem, s>>>(a);
        return cudaGetLastError();
    }
};

} // namespace kernel
} // namespace qmlp
