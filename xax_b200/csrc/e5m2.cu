// float8_e5m2 for the free functions of xax/nn/fp8.py: quantize (:97-120), dequantize (:123-138) and, with
// xaxb_gemm_fp8_formats, fp8_matmul (:347-378) and quantize_dequantize (:141-162) called with
// fp8_dtype=float8_e5m2.  The transformer path quantises to e4m3 only and has its own fused kernels
// (quantize.cu); these are plain streaming kernels with the same arithmetic as those, in the bf16 compute dtype:
//   q = e5m2( clip( bf16(x * s), +-57344 ) ),  s = bf16(given scale)  or  bf16(57344 / max(amax, bf16(1e-12))).
// NaN becomes 0x7E / 0xFE (the quiet NaN the reference's cast produces), infinities clip to +-57344.
#include "common.cuh"
#include "quant_device.cuh"

namespace xaxb {

constexpr float kE5M2Max = 57344.0f;

__device__ __forceinline__ float scaled_clipped_e5m2(float x, float s) {
  const float p = bf16_round(x * s);
  return (p != p) ? p : fminf(fmaxf(p, -kE5M2Max), kE5M2Max);
}

__device__ __forceinline__ uint32_t e5m2x2(float lo, float hi) {
  // cvt.rn.satfinite.e5m2x2.f32: first source operand -> upper byte, second -> lower byte.
  uint16_t r;
  asm("cvt.rn.satfinite.e5m2x2.f32 %0, %1, %2;" : "=h"(r) : "f"(hi), "f"(lo));
  uint32_t v = r;
  if (lo != lo) v = (v & 0xFF00u) | 0x7Eu | ((__float_as_uint(lo) >> 24) & 0x80u);
  if (hi != hi) v = (v & 0x00FFu) | ((0x7Eu | ((__float_as_uint(hi) >> 24) & 0x80u)) << 8);
  return v;
}

__device__ __forceinline__ uint2 quantize8_e5m2(const uint4 v, float s) {
  float f[8];
  unpack8(v, f);
  uint2 r;
  r.x = e5m2x2(scaled_clipped_e5m2(f[0], s), scaled_clipped_e5m2(f[1], s)) |
        (e5m2x2(scaled_clipped_e5m2(f[2], s), scaled_clipped_e5m2(f[3], s)) << 16);
  r.y = e5m2x2(scaled_clipped_e5m2(f[4], s), scaled_clipped_e5m2(f[5], s)) |
        (e5m2x2(scaled_clipped_e5m2(f[6], s), scaled_clipped_e5m2(f[7], s)) << 16);
  return r;
}

// grid (x, groups): group g is vec_per_group consecutive 16-byte pieces.  The scale of a group is the given
// scalar (scale_in, shared by all groups) or derived from the group's amax.
__global__ void __launch_bounds__(256) e5m2_cast_kernel(const uint4* __restrict__ x, int64_t vec_per_group,
                                                        int64_t group_rows, const float* __restrict__ scale_in,
                                                        const float* __restrict__ amax, uint2* __restrict__ q,
                                                        float* __restrict__ scale, float* __restrict__ inv_scale) {
  pdl_trigger();
  pdl_wait();
  const int64_t g = blockIdx.y;
  float s;
  if (scale_in) {
    s = bf16_round(*scale_in);
  } else {
    const float a = amax[g];
    const float floor_v = bf16_round(1e-12f);
    const float denom = (a != a) ? a : fmaxf(a, floor_v);
    s = bf16_round(kE5M2Max / denom);
  }
  const uint4* xg = x + g * vec_per_group;
  uint2* qg = q + g * vec_per_group;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < vec_per_group; i += (int64_t)gridDim.x * blockDim.x)
    qg[i] = quantize8_e5m2(__ldg(xg + i), s);
  if (scale && blockIdx.x == 0)
    for (int64_t r = threadIdx.x; r < group_rows; r += blockDim.x) {
      scale[g * group_rows + r] = s;
      inv_scale[g * group_rows + r] = 1.0f / s;
    }
}

template <bool OUT_BF16>
__global__ void __launch_bounds__(256) e5m2_dequantize_kernel(const uint2* __restrict__ q, int64_t vec_per_row,
                                                              int64_t n_vec, const float* __restrict__ scale,
                                                              int scale_stride, void* __restrict__ out) {
  pdl_trigger();
  pdl_wait();
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n_vec; i += (int64_t)gridDim.x * blockDim.x) {
    const float s_raw = scale[(i / vec_per_row) * scale_stride];
    const float s = OUT_BF16 ? bf16_round(s_raw) : s_raw;
    const uint2 v = __ldg(q + i);
    const uint32_t w[2] = {v.x, v.y};
    float f[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      // an e5m2 byte is the upper byte of the half with the same value
      const uint32_t byte = (w[k >> 2] >> ((k & 3) * 8)) & 0xFFu;
      f[k] = __half2float(__ushort_as_half((unsigned short)(byte << 8))) / s;
    }
    if (OUT_BF16) {
      reinterpret_cast<uint4*>(out)[i] = pack8(f);
    } else {
      reinterpret_cast<float4*>(out)[2 * i] = make_float4(f[0], f[1], f[2], f[3]);
      reinterpret_cast<float4*>(out)[2 * i + 1] = make_float4(f[4], f[5], f[6], f[7]);
    }
  }
}

}  // namespace xaxb

using namespace xaxb;

extern "C" {

int xaxb_quantize_e5m2(xaxb_ctx* ctx, void* stream, const void* x_bf16, int64_t rows, int64_t cols, int64_t group_rows,
                       const float* scale_in, const float* group_amax, void* q_e5m2, float* scale, float* inv_scale) {
  if (!ctx || !x_bf16 || !q_e5m2 || rows <= 0 || cols <= 0 || cols % 8 != 0 ||
      ((reinterpret_cast<uintptr_t>(x_bf16) | reinterpret_cast<uintptr_t>(q_e5m2)) & 15)) {
    set_last_error("quantize_e5m2: null pointer, cols (%lld) not a positive multiple of 8, or misaligned buffers",
                   (long long)cols);
    return XAXB_BAD_ARGUMENT;
  }
  if ((scale_in == nullptr) == (group_amax == nullptr) || (scale != nullptr) != (inv_scale != nullptr)) {
    set_last_error("quantize_e5m2: give exactly one of scale_in / group_amax, and scale with inv_scale");
    return XAXB_BAD_ARGUMENT;
  }
  if (group_rows <= 0 || rows % group_rows != 0 || rows / group_rows > 65535) {
    set_last_error("quantize_e5m2: group_rows (%lld) must divide rows (%lld) into at most 65535 groups",
                   (long long)group_rows, (long long)rows);
    return XAXB_BAD_ARGUMENT;
  }
  const Ctx* c = reinterpret_cast<const Ctx*>(ctx);
  const int64_t groups = rows / group_rows;
  const int64_t vec_per_group = group_rows * cols / 8;
  int64_t bx = (vec_per_group + 255) / 256;
  const int64_t cap = ((int64_t)c->num_sms * 8 + groups - 1) / groups;
  if (bx > cap) bx = cap;
  launch_kernel(e5m2_cast_kernel, dim3((unsigned)bx, (unsigned)groups), dim3(256), 0, static_cast<cudaStream_t>(stream), 1,
                static_cast<const uint4*>(x_bf16), vec_per_group, group_rows, scale_in, group_amax,
                static_cast<uint2*>(q_e5m2), scale, inv_scale);
  return check_launch("e5m2_cast_kernel");
}

int xaxb_dequantize_e5m2(xaxb_ctx* ctx, void* stream, const void* q_e5m2, int64_t rows, int64_t cols, const float* scale,
                         int scale_stride, int out_is_bf16, void* out) {
  if (!ctx || !q_e5m2 || !scale || !out || rows <= 0 || cols <= 0 || cols % 8 != 0 ||
      (scale_stride != 0 && scale_stride != 1) ||
      ((reinterpret_cast<uintptr_t>(q_e5m2) & 7) | (reinterpret_cast<uintptr_t>(out) & 15))) {
    set_last_error("dequantize_e5m2: null pointer, cols not a positive multiple of 8, scale_stride not 0/1, or "
                   "misaligned buffers");
    return XAXB_BAD_ARGUMENT;
  }
  const Ctx* c = reinterpret_cast<const Ctx*>(ctx);
  const int64_t n_vec = rows * cols / 8;
  int64_t grid = (n_vec + 255) / 256;
  if (grid > (int64_t)c->num_sms * 8) grid = (int64_t)c->num_sms * 8;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (out_is_bf16)
    launch_kernel(e5m2_dequantize_kernel<true>, dim3((unsigned)grid), dim3(256), 0, s, 1,
                  static_cast<const uint2*>(q_e5m2), cols / 8, n_vec, scale, scale_stride, out);
  else
    launch_kernel(e5m2_dequantize_kernel<false>, dim3((unsigned)grid), dim3(256), 0, s, 1,
                  static_cast<const uint2*>(q_e5m2), cols / 8, n_vec, scale, scale_stride, out);
  return check_launch("e5m2_dequantize_kernel");
}

}  // extern "C"
