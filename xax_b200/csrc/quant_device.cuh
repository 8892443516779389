// Device helpers shared by the quantising kernels (stand-alone cast, RMSNorm and SiLU*up
// with a fused cast): bf16 magnitude max on packed words, the reference's scale formula,
// and the bf16 -> e4m3 conversion with its intermediate bf16 rounding.
#pragma once

#include "common.cuh"

namespace xaxb {

// max over the magnitudes (bf16 bit patterns with the sign cleared) of two packed pairs.
// Unsigned order on the magnitude bits equals numeric order and puts NaN above infinity,
// so a NaN input propagates to the result as jnp.max does.
__device__ __forceinline__ uint32_t absmax_bits2(uint32_t m16, uint32_t packed) {
  const uint32_t a = packed & 0x7FFF7FFFu;
  const uint32_t hi = a >> 16, lo = a & 0xFFFFu;
  return max(m16, max(hi, lo));
}

__device__ __forceinline__ uint32_t absmax_bits8(uint32_t m16, const uint4 v) {
  const uint32_t a = __vmaxu2(__vmaxu2(v.x & 0x7FFF7FFFu, v.y & 0x7FFF7FFFu),
                              __vmaxu2(v.z & 0x7FFF7FFFu, v.w & 0x7FFF7FFFu));
  return max(m16, max(a >> 16, a & 0xFFFFu));
}

// Block-wide max of a 32-bit unsigned value; every thread gets the result.
__device__ __forceinline__ uint32_t block_max_u32(uint32_t v) {
  __shared__ uint32_t warp_vals[32];
  __shared__ uint32_t result;
  for (int o = 16; o > 0; o >>= 1) v = max(v, __shfl_xor_sync(0xffffffffu, v, o));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();  // protects warp_vals / result across repeated calls
  if (lane == 0) warp_vals[warp] = v;
  __syncthreads();
  if (warp == 0) {
    const int nw = (blockDim.x + 31) >> 5;
    uint32_t w = lane < nw ? warp_vals[lane] : 0u;
    for (int o = 16; o > 0; o >>= 1) w = max(w, __shfl_xor_sync(0xffffffffu, w, o));
    if (lane == 0) result = w;
  }
  __syncthreads();
  return result;
}

__device__ __forceinline__ float block_sum_f32(float v) {
  __shared__ float warp_vals[32];
  __shared__ float result;
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();
  if (lane == 0) warp_vals[warp] = v;
  __syncthreads();
  if (warp == 0) {
    const int nw = (blockDim.x + 31) >> 5;
    float w = lane < nw ? warp_vals[lane] : 0.0f;
    for (int o = 16; o > 0; o >>= 1) w += __shfl_xor_sync(0xffffffffu, w, o);
    if (lane == 0) result = w;
  }
  __syncthreads();
  return result;
}

// s = bf16(448 / max(amax, bf16(1e-12))): the whole expression is bf16 in the reference
// (the divisor floor is a weak Python scalar), and a NaN amax gives a NaN scale.
__device__ __forceinline__ float current_scale_from_amax(float amax_bf16_value) {
  const float floor_v = bf16_round(1e-12f);
  const float denom = (amax_bf16_value != amax_bf16_value) ? amax_bf16_value : fmaxf(amax_bf16_value, floor_v);
  return bf16_round(448.0f / denom);
}

// One value: bf16(x * s) clipped to +-448 -> e4m3 byte.  NaN keeps being NaN (0x7F).
__device__ __forceinline__ float scaled_clipped(float x, float s) {
  const float p = bf16_round(x * s);
  return (p != p) ? p : fminf(fmaxf(p, -448.0f), 448.0f);
}

__device__ __forceinline__ uint32_t e4m3x2(float lo, float hi) {
  // cvt.rn.satfinite.e4m3x2.f32: first source operand -> upper byte, second -> lower byte.
  uint16_t r;
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(r) : "f"(hi), "f"(lo));
  return r;
}

__device__ __forceinline__ uint32_t quantize2(uint32_t packed_bf16x2, float s) {
  const float lo = scaled_clipped(bf16_bits_to_float(packed_bf16x2 & 0xFFFFu), s);
  const float hi = scaled_clipped(bf16_bits_to_float(packed_bf16x2 >> 16), s);
  return e4m3x2(lo, hi);
}

// Two bf16 values at once: the product is taken and rounded in bf16 by the packed multiply (the exact product
// of two bf16 values fits float32, so one rounding either way: the same bits as bf16(float(x) * float(s))),
// clipped by NaN-propagating packed min / max, widened by a shift and a mask, and cast.  Half the instructions
// of the scalar route; the cast of 8192 x 8192 was bound by them, not by memory.
__device__ __forceinline__ uint32_t quantize2_packed(uint32_t packed_bf16x2, uint32_t s_bf16x2) {
  uint32_t p;
  asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(p) : "r"(packed_bf16x2), "r"(s_bf16x2));
  asm("min.NaN.bf16x2 %0, %1, %2;" : "=r"(p) : "r"(p), "r"(0x43E043E0u));  // +448
  asm("max.NaN.bf16x2 %0, %1, %2;" : "=r"(p) : "r"(p), "r"(0xC3E0C3E0u));  // -448
  return e4m3x2(__uint_as_float(p << 16), __uint_as_float(p & 0xFFFF0000u));
}

// s must already be rounded to bf16 (every caller multiplies by bf16(scale)).
__device__ __forceinline__ uint2 quantize8_packed(const uint4 v, float s) {
  const uint32_t sb = __float_as_uint(s) >> 16, s2 = sb | (sb << 16);
  uint2 r;
  r.x = quantize2_packed(v.x, s2) | (quantize2_packed(v.y, s2) << 16);
  r.y = quantize2_packed(v.z, s2) | (quantize2_packed(v.w, s2) << 16);
  return r;
}

__device__ __forceinline__ uint2 quantize8(const uint4 v, float s) {
  uint2 r;
  r.x = quantize2(v.x, s) | (quantize2(v.y, s) << 16);
  r.y = quantize2(v.z, s) | (quantize2(v.w, s) << 16);
  return r;
}

// Eight float values already rounded to bf16 -> 8 e4m3 bytes.
__device__ __forceinline__ uint2 quantize8f(const float (&y)[8], float s) {
  uint2 r;
  r.x = e4m3x2(scaled_clipped(y[0], s), scaled_clipped(y[1], s)) |
        (e4m3x2(scaled_clipped(y[2], s), scaled_clipped(y[3], s)) << 16);
  r.y = e4m3x2(scaled_clipped(y[4], s), scaled_clipped(y[5], s)) |
        (e4m3x2(scaled_clipped(y[6], s), scaled_clipped(y[7], s)) << 16);
  return r;
}

__device__ __forceinline__ void unpack8(const uint4 v, float (&f)[8]) {
  f[0] = bf16_bits_to_float(v.x & 0xFFFFu);
  f[1] = bf16_bits_to_float(v.x >> 16);
  f[2] = bf16_bits_to_float(v.y & 0xFFFFu);
  f[3] = bf16_bits_to_float(v.y >> 16);
  f[4] = bf16_bits_to_float(v.z & 0xFFFFu);
  f[5] = bf16_bits_to_float(v.z >> 16);
  f[6] = bf16_bits_to_float(v.w & 0xFFFFu);
  f[7] = bf16_bits_to_float(v.w >> 16);
}

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  const uint32_t l = __bfloat16_as_ushort(__float2bfloat16_rn(lo));
  const uint32_t h = __bfloat16_as_ushort(__float2bfloat16_rn(hi));
  return l | (h << 16);
}

__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  uint4 r;
  r.x = pack_bf16x2(f[0], f[1]);
  r.y = pack_bf16x2(f[2], f[3]);
  r.z = pack_bf16x2(f[4], f[5]);
  r.w = pack_bf16x2(f[6], f[7]);
  return r;
}

// RoPE, "concatenated" style (xax/arch/attention.py:510-515), on eight pairs (i, i + D/2): a holds
// x[i .. i+7], b holds x[i + D/2 .. i + D/2 + 7], c / s the cos / sin values of those eight
// frequencies.  Every product and every sum is rounded to bf16 as the reference's bf16 ops do.
__device__ __forceinline__ void rope_rotate_pieces(const uint4 a, const uint4 b, const uint4 c, const uint4 s, uint4& o1,
                                                   uint4& o2) {
  // Packed bf16 arithmetic, two pairs per instruction; the _rn forms are never contracted into a fused
  // multiply-add.  A bf16 sum of two bf16 values rounds once where float32-then-bf16 rounds twice, but the
  // first of those two roundings only happens for operands more than 2^16 apart, where the sum is nowhere
  // near a bf16 tie: the bits are the same.
  const __nv_bfloat162* aw = reinterpret_cast<const __nv_bfloat162*>(&a);
  const __nv_bfloat162* bw = reinterpret_cast<const __nv_bfloat162*>(&b);
  const __nv_bfloat162* cw = reinterpret_cast<const __nv_bfloat162*>(&c);
  const __nv_bfloat162* sw = reinterpret_cast<const __nv_bfloat162*>(&s);
  uint4 r1, r2;
  __nv_bfloat162* w1 = reinterpret_cast<__nv_bfloat162*>(&r1);
  __nv_bfloat162* w2 = reinterpret_cast<__nv_bfloat162*>(&r2);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    w1[j] = __hsub2_rn(__hmul2_rn(aw[j], cw[j]), __hmul2_rn(bw[j], sw[j]));
    w2[j] = __hadd2_rn(__hmul2_rn(bw[j], cw[j]), __hmul2_rn(aw[j], sw[j]));
  }
  o1 = r1;
  o2 = r2;
}

// magnitude bits (bf16, sign cleared) of a float that already holds a bf16 value
__device__ __forceinline__ uint32_t mag_bits16(float v) { return (__float_as_uint(v) >> 16) & 0x7FFFu; }

}  // namespace xaxb
