// Device helpers shared by the MLX Q4/Q8 kernels: streaming loads, bf16
// widening/narrowing with the reference's store rule, nibble-to-float tricks and
// the activations of kernels/act.h (reference project path).
#pragma once

#include <cuda_runtime.h>

#include <cstdint>

namespace tessl {
namespace dev {

/// 16-byte read-only load that does not allocate in L1: weights are touched
/// exactly once per launch.
__device__ __forceinline__ uint4 ldg_stream16(const void *p)
{
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

__device__ __forceinline__ uint32_t ldg_stream4(const void *p)
{
    uint32_t v;
    asm volatile("ld.global.nc.L1::no_allocate.u32 %0, [%1];" : "=r"(v) : "l"(p));
    return v;
}

/// The two bf16 halves of a word, widened (a bf16 is the top half of an f32).
__device__ __forceinline__ float bf16_lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t w) { return __uint_as_float(w & 0xffff0000u); }

/// f32 -> bf16 bits as the reference's device cast stores them
/// (`f32_to_bf16_bits_gpu`, src/tensor.rs:815-831 of the reference project):
/// any NaN becomes 0x7fc0, an f32 subnormal flushes to a zero of its sign,
/// everything else rounds to nearest even.
__device__ __forceinline__ uint16_t f32_to_bf16_store(float x)
{
    const uint32_t bits = __float_as_uint(x);
    const uint32_t mag = bits & 0x7fffffffu;
    if (mag > 0x7f800000u) return 0x7fc0u;
    if (mag < 0x00800000u) return (uint16_t)((bits >> 16) & 0x8000u);
    return (uint16_t)((bits + 0x7fffu + ((bits >> 16) & 1u)) >> 16);
}

/// Byte `B` of `bytes` (each byte one nibble value 0..15) as the float
/// 128 + q: the byte lands in mantissa bits 16..23 under exponent 2^7. One
/// PRMT, no integer-to-float conversion.
template <int B>
__device__ __forceinline__ float nib_byte_to_f128(uint32_t bytes)
{
    return __uint_as_float(__byte_perm(bytes, 0x00004300u, 0x5044u | (B << 8)));
}

/// kernels/act.h:36-46 (reference project): sigmoid through e = exp(-|x|) so
/// no intermediate overflows, then x * sigmoid(x).
__device__ __forceinline__ float silu(float x)
{
    const float e = expf(-fabsf(x));
    const float r = __fdiv_rn(1.0f, 1.0f + e);
    return x * (x >= 0.0f ? r : e * r);
}

/// kernels/act.h:24-30 (reference project): tanh-approximate GELU with the
/// cubic's input clamped to +-20 and the tanh argument to +-10; the outer
/// factor stays the original x.
__device__ __forceinline__ float gelu_pytorch_tanh(float x)
{
    const float xc = fminf(fmaxf(x, -20.0f), 20.0f);
    const float x3 = xc * xc * xc;
    const float inner = 0.7978845608028654f * (xc + 0.044715f * x3);
    const float t = tanhf(fminf(fmaxf(inner, -10.0f), 10.0f));
    return 0.5f * x * (1.0f + t);
}

__device__ __forceinline__ float warp_sum(float v)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

}  // namespace dev
}  // namespace tessl
