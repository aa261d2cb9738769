// Activation functors used by the fused kernels.
//
// The reference turns every activation (id, forward snippet, adjoint snippet) into
//   struct id { static __device__ half forward(half x); static __device__ half adjoint(half x, half adjz); };
// (src_cpp/src/activation.cpp:13-40). The fused kernels here work on half2 pairs, so a functor exposes
// forward2 / adjoint2. User snippets are wrapped by ScalarActivation; the four built-ins of
// src_cpp/include/qmlp/builtin-activations.json:1-21 have hand-written half2 forms with the same semantics.
#pragma once
#include <cuda_fp16.h>
#include <stdint.h>
#include <type_traits>

// helpers user snippets may reference (src_cpp/include/qmlp/kernels/common.cuh:16-19)
__device__ __forceinline__ half hZERO() { return __ushort_as_half(0); }

namespace qmlp {
namespace kernel {

template <class A>
struct ScalarActivation {
    static __device__ __forceinline__ __half2 forward2(__half2 x)
    {
        return __halves2half2(A::forward(__low2half(x)), A::forward(__high2half(x)));
    }
    static __device__ __forceinline__ __half2 adjoint2(__half2 x, __half2 adjz)
    {
        return __halves2half2(A::adjoint(__low2half(x), __low2half(adjz)),
                              A::adjoint(__high2half(x), __high2half(adjz)));
    }
    static __device__ __forceinline__ half forward(half x) { return A::forward(x); }
    static __device__ __forceinline__ half adjoint(half x, half adjz) { return A::adjoint(x, adjz); }
    // activation of two fp32 pre-activations, result as half2: round to half, then the half snippet
    static __device__ __forceinline__ __half2 forward_f32x2(float a, float b) { return forward2(__floats2half2_rn(a, b)); }
};

__device__ __forceinline__ __half2 select_gt0(__half2 x, __half2 ifTrue, __half2 ifFalse)
{
    // per lane: x > 0 ? ifTrue : ifFalse (false for NaN, like __hgt)
    uint32_t m = __hgt2_mask(x, __float2half2_rn(0.f));
    uint32_t t = *reinterpret_cast<uint32_t*>(&ifTrue);
    uint32_t f = *reinterpret_cast<uint32_t*>(&ifFalse);
    uint32_t r = (t & m) | (f & ~m);
    return *reinterpret_cast<__half2*>(&r);
}

// "z = __hgt(x, hZERO()) ? x : hZERO()" / "adjx = __hgt(x, hZERO()) ? adjz : hZERO()"
struct BuiltinRelu {
    // max(x, 0) returns the non-NaN operand, i.e. 0 for NaN, like the comparison form
    static __device__ __forceinline__ __half2 forward2(__half2 x) { return __hmax2(x, __float2half2_rn(0.f)); }
    static __device__ __forceinline__ __half2 adjoint2(__half2 x, __half2 adjz) { return select_gt0(x, adjz, __float2half2_rn(0.f)); }
    static __device__ __forceinline__ half forward(half x) { return __hgt(x, hZERO()) ? x : hZERO(); }
    static __device__ __forceinline__ half adjoint(half x, half adjz) { return __hgt(x, hZERO()) ? adjz : hZERO(); }
    // rounding and clamping in one conversion instruction (a NaN input stays NaN here; the comparison form gives 0)
    static __device__ __forceinline__ __half2 forward_f32x2(float a, float b)
    {
        uint32_t r;
        asm("cvt.rn.relu.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(b), "f"(a));
        return *reinterpret_cast<__half2*>(&r);
    }
};

// "z = __hgt(x, hZERO()) ? x : __hsub(hexp(x), 1)" / "adjx = __hgt(x, hZERO()) ? adjz : __hmul(adjz, hexp(x))"
struct BuiltinCelu {
    // exp(x) = 2^(x * log2 e) on the half2 special-function path; only used for x <= 0, where the fp16 rounding of
    // the product costs less than one fp16 ulp of the result
    static __device__ __forceinline__ __half2 fast_exp2(__half2 x)
    {
        return h2exp2(__hmul2(x, __float2half2_rn(1.4426950408889634f)));
    }
    static __device__ __forceinline__ __half2 forward2(__half2 x)
    {
        return select_gt0(x, x, __hsub2(fast_exp2(x), __float2half2_rn(1.0f)));
    }
    static __device__ __forceinline__ __half2 adjoint2(__half2 x, __half2 adjz)
    {
        return select_gt0(x, adjz, __hmul2(adjz, fast_exp2(x)));
    }
    static __device__ __forceinline__ half forward(half x) { return __hgt(x, hZERO()) ? x : __hsub(hexp(x), __float2half(1.0f)); }
    static __device__ __forceinline__ half adjoint(half x, half adjz) { return __hgt(x, hZERO()) ? adjz : __hmul(adjz, hexp(x)); }
    static __device__ __forceinline__ float celu_f32(float x)
    {
        float e;
        asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(x * 1.4426950408889634f));
        return x > 0.f ? x : e - 1.f;
    }
    // (a half2 form from the rounding on - pack, ex2.approx.f16x2, subtract, select - has fewer instructions but measured
    // 5 % slower in the tcgen05 epilogue and less accurate than the fp32 form)
    static __device__ __forceinline__ __half2 forward_f32x2(float a, float b) { return __floats2half2_rn(celu_f32(a), celu_f32(b)); }
};

// "z = hsin(x)" / "adjx = __hmul(hcos(x), adjz)"
struct BuiltinSine {
    // fp32 special-function unit (sin.approx / cos.approx, absolute error ~1e-6 for the |x| an fp16 pre-activation can
    // hold with useful precision), rounded once to half
    static __device__ __forceinline__ __half2 forward2(__half2 x)
    {
        const float2 f = __half22float2(x);
        return __floats2half2_rn(__sinf(f.x), __sinf(f.y));
    }
    static __device__ __forceinline__ __half2 adjoint2(__half2 x, __half2 adjz)
    {
        const float2 f = __half22float2(x);
        return __hmul2(__floats2half2_rn(__cosf(f.x), __cosf(f.y)), adjz);
    }
    static __device__ __forceinline__ half forward(half x) { return hsin(x); }
    static __device__ __forceinline__ half adjoint(half x, half adjz) { return __hmul(hcos(x), adjz); }
    static __device__ __forceinline__ __half2 forward_f32x2(float a, float b) { return __floats2half2_rn(__sinf(a), __sinf(b)); }
};

// "z = x" / "adjx = adjz"
struct BuiltinIdentity {
    static __device__ __forceinline__ __half2 forward2(__half2 x) { return x; }
    static __device__ __forceinline__ __half2 adjoint2(__half2, __half2 adjz) { return adjz; }
    static __device__ __forceinline__ half forward(half x) { return x; }
    static __device__ __forceinline__ half adjoint(half, half adjz) { return adjz; }
    static __device__ __forceinline__ __half2 forward_f32x2(float a, float b) { return __floats2half2_rn(a, b); }
};

// ---- per-channel activation arrays -----------------------------------------------------------------------------------
// A layer may name one activation per output channel ("activation": [...], src_cpp/src/fused_network.cpp:106-125; the
// reference parses such arrays and then refuses to generate code for them, :447). The generated functor of such a layer
// declares PER_CHANNEL and takes the channel of the first of the two values; the kernels call through these helpers,
// which drop the channel for ordinary functors.
template <class A, class = void>
struct is_per_channel : std::false_type {};
template <class A>
struct is_per_channel<A, std::void_t<decltype(A::PER_CHANNEL)>> : std::true_type {};

template <class A>
__device__ __forceinline__ __half2 act_forward2(__half2 x, int channel)
{
    if constexpr (is_per_channel<A>::value) return A::forward2c(x, channel);
    else return A::forward2(x);
}
template <class A>
__device__ __forceinline__ __half2 act_adjoint2(__half2 x, __half2 adjz, int channel)
{
    if constexpr (is_per_channel<A>::value) return A::adjoint2c(x, adjz, channel);
    else return A::adjoint2(x, adjz);
}
template <class A>
__device__ __forceinline__ __half2 act_forward_f32x2(float a, float b, int channel)
{
    if constexpr (is_per_channel<A>::value) return A::forward2c(__floats2half2_rn(a, b), channel);
    else return A::forward_f32x2(a, b);
}

// both values belong to the same channel (fragments that pair two points of one channel)
template <class A>
__device__ __forceinline__ __half2 act_forward2_same_channel(__half2 x, int channel)
{
    if constexpr (is_per_channel<A>::value) return A::forward2s(x, channel);
    else return A::forward2(x);
}

// Base of a generated per-channel functor: D supplies forward1(half, channel) and adjoint1(half, half, channel).
template <class D>
struct PerChannelActivation {
    static constexpr bool PER_CHANNEL = true;
    static __device__ __forceinline__ __half2 forward2c(__half2 x, int c)
    {
        return __halves2half2(D::forward1(__low2half(x), c), D::forward1(__high2half(x), c + 1));
    }
    static __device__ __forceinline__ __half2 forward2s(__half2 x, int c)
    {
        return __halves2half2(D::forward1(__low2half(x), c), D::forward1(__high2half(x), c));
    }
    static __device__ __forceinline__ __half2 adjoint2c(__half2 x, __half2 adjz, int c)
    {
        return __halves2half2(D::adjoint1(__low2half(x), __low2half(adjz), c),
                              D::adjoint1(__high2half(x), __high2half(adjz), c + 1));
    }
};

} // namespace kernel
} // namespace qmlp
