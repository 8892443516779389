// Small bandwidth kernels on the path (RMSNorm, SiLU*up, embedding gather, arg-max, RoPE +
// KV-cache append) and the CUDA-core check kernels.  bf16 intermediates are rounded where
// the reference's bf16 ops round, so outputs match the oracle except for float32 summation
// order.
#include "common.cuh"
#include "quant_device.cuh"
#include "tp_device.cuh"

namespace xaxb {

// ---------------------------------------------------------------------------------------
// RMSNorm: x / sqrt(mean(x^2) + eps) * w, one CTA per row, optional fused per-token cast.

__device__ __forceinline__ void rmsnorm8(const uint4 xv, const uint4 wv, float n, float (&y)[8]) {
  float x[8], w[8];
  unpack8(xv, x);
  unpack8(wv, w);
#pragma unroll
  for (int j = 0; j < 8; ++j) y[j] = bf16_round(bf16_round(x[j] / n) * w[j]);
}

__global__ void __launch_bounds__(256) rmsnorm_kernel(const uint4* __restrict__ x, const uint4* __restrict__ w,
                                                      float eps, int64_t vec, uint4* __restrict__ y,
                                                      uint2* __restrict__ q, float* __restrict__ scale,
                                                      float* __restrict__ inv_scale,
                                                      unsigned int* __restrict__ group_amax, int64_t group_rows) {
  pdl_trigger();
  pdl_wait();
  const int64_t row = blockIdx.x;
  const uint4* xr = x + row * vec;
  float acc = 0.0f;
  for (int64_t i = threadIdx.x; i < vec; i += blockDim.x) {
    float f[8];
    unpack8(__ldg(xr + i), f);
#pragma unroll
    for (int j = 0; j < 8; ++j) acc += bf16_round(f[j] * f[j]);
  }
  const float total = block_sum_f32(acc);
  const float mean = bf16_round(total / (float)(vec * 8));
  const float n = bf16_round(sqrtf(bf16_round(mean + bf16_round(eps))));

  uint32_t m = 0;
  for (int64_t i = threadIdx.x; i < vec; i += blockDim.x) {
    float yv[8];
    rmsnorm8(__ldg(xr + i), __ldg(w + i), n, yv);
    if (y) y[row * vec + i] = pack8(yv);
#pragma unroll
    for (int j = 0; j < 8; ++j) m = max(m, mag_bits16(yv[j]));
  }
  if (!q && !group_amax) return;
  const uint32_t row_bits = block_max_u32(m);
  if (group_amax && threadIdx.x == 0) atomicMax(group_amax + row / group_rows, row_bits << 16);
  if (!q) return;
  const float s = current_scale_from_amax(bf16_bits_to_float(row_bits));
  for (int64_t i = threadIdx.x; i < vec; i += blockDim.x) {
    float yv[8];
    rmsnorm8(__ldg(xr + i), __ldg(w + i), n, yv);
    q[row * vec + i] = quantize8f(yv, s);
  }
  if (threadIdx.x == 0) {
    scale[row] = s;
    inv_scale[row] = 1.0f / s;
  }
}

// ---------------------------------------------------------------------------------------
// h = bf16(silu(g) * u), silu(g) = bf16(g * bf16(sigmoid(g)))

__device__ __forceinline__ void silu_mul8(const uint4 gv, const uint4 uv, float (&h)[8]) {
  float g[8], u[8];
  unpack8(gv, g);
  unpack8(uv, u);
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const float sig = bf16_round(1.0f / (1.0f + expf(-g[j])));
    h[j] = bf16_round(bf16_round(g[j] * sig) * u[j]);
  }
}

__global__ void __launch_bounds__(1024) silu_mul_kernel(const uint4* __restrict__ gate, const uint4* __restrict__ up,
                                                       int64_t ld_vec, int64_t vec, uint4* __restrict__ h,
                                                       uint2* __restrict__ q, float* __restrict__ scale,
                                                       float* __restrict__ inv_scale,
                                                       unsigned int* __restrict__ group_amax, int64_t group_rows,
                                                       const TpRowMax tp, int* d_status) {
  pdl_trigger();
  pdl_wait();
  __shared__ uint32_t s_tp[2];
  const int64_t row = blockIdx.x;
  const uint4* gr = gate + row * ld_vec;
  const uint4* ur = up + row * ld_vec;
  uint32_t m = 0;
  for (int64_t i = threadIdx.x; i < vec; i += blockDim.x) {
    float hv[8];
    silu_mul8(__ldg(gr + i), __ldg(ur + i), hv);
    if (h) h[row * vec + i] = pack8(hv);
#pragma unroll
    for (int j = 0; j < 8; ++j) m = max(m, mag_bits16(hv[j]));
  }
  if (!q && !group_amax) return;
  uint32_t row_bits = block_max_u32(m);
  // tensor-parallel runs: the row continues on the other ranks (the down projection's input is
  // split along its width), so the amax that sets the scale is the maximum over ranks
  if (tp.world > 1) row_bits = tp_cta_max_u32(tp, (int)row, row_bits, s_tp, d_status, kSiteTpSilu);
  if (group_amax && threadIdx.x == 0) atomicMax(group_amax + row / group_rows, row_bits << 16);
  if (!q) return;
  const float s = current_scale_from_amax(bf16_bits_to_float(row_bits));
  for (int64_t i = threadIdx.x; i < vec; i += blockDim.x) {
    float hv[8];
    silu_mul8(__ldg(gr + i), __ldg(ur + i), hv);
    q[row * vec + i] = quantize8f(hv, s);
  }
  if (threadIdx.x == 0) {
    scale[row] = s;
    inv_scale[row] = 1.0f / s;
  }
}


// Register-resident variant for rows of up to NT * VPT * 8 elements: the row is read from
// global memory once and stays in registers through the three phases (sum of squares,
// normalise + amax, cast).  With few rows (a decode step) a CTA is alone on its SM, and what bounds
// it is the dependent-instruction latency of its own warps: such launches spread a row over more
// threads (NT = 512 or 1024, one 16-byte piece each).
template <int VPT, int NT = 256>
__global__ void __launch_bounds__(NT) rmsnorm_reg_kernel(const uint4* __restrict__ x, const uint4* __restrict__ w,
                                                          float eps, int vec, uint4* __restrict__ y,
                                                          uint2* __restrict__ q, float* __restrict__ scale,
                                                          float* __restrict__ inv_scale,
                                                          unsigned int* __restrict__ group_amax, int64_t group_rows) {
  pdl_trigger();
  pdl_wait();
  const int64_t row = blockIdx.x;
  const uint4* xr = x + row * vec;
  float v[VPT][8];
  float acc = 0.0f;
#pragma unroll
  for (int k = 0; k < VPT; ++k) {
    const int i = threadIdx.x + k * NT;
    if (i < vec) {
      unpack8(__ldg(xr + i), v[k]);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc += bf16_round(v[k][j] * v[k][j]);
    }
  }
  const float total = block_sum_f32(acc);
  const float mean = bf16_round(total / (float)(vec * 8));
  const float n = bf16_round(sqrtf(bf16_round(mean + bf16_round(eps))));
  uint32_t m = 0;
#pragma unroll
  for (int k = 0; k < VPT; ++k) {
    const int i = threadIdx.x + k * NT;
    if (i < vec) {
      float wv[8];
      unpack8(__ldg(w + i), wv);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        v[k][j] = bf16_round(bf16_round(v[k][j] / n) * wv[j]);
        m = max(m, mag_bits16(v[k][j]));
      }
      if (y) y[row * vec + i] = pack8(v[k]);
    }
  }
  if (!q && !group_amax) return;
  const uint32_t row_bits = block_max_u32(m);
  if (group_amax && threadIdx.x == 0) atomicMax(group_amax + row / group_rows, row_bits << 16);
  if (!q) return;
  const float s = current_scale_from_amax(bf16_bits_to_float(row_bits));
#pragma unroll
  for (int k = 0; k < VPT; ++k) {
    const int i = threadIdx.x + k * NT;
    if (i < vec) q[row * vec + i] = quantize8f(v[k], s);
  }
  if (threadIdx.x == 0) {
    scale[row] = s;
    inv_scale[row] = 1.0f / s;
  }
}

// SiLU*up with the row spread over a thread-block cluster of C CTAs (C <= 8): every CTA keeps
// its slice of h in registers, the row's amax is the max of the C CTAs' partial maxima read
// through distributed shared memory, and the cast happens from registers.  gate and up are read
// once and h never travels through global memory unless the caller asks for it.
__device__ __forceinline__ uint32_t ld_dsmem_u32(uint32_t local_smem_addr, uint32_t cta) {
  uint32_t remote, v;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_smem_addr), "r"(cta));
  asm volatile("ld.shared::cluster.u32 %0, [%1];" : "=r"(v) : "r"(remote) : "memory");
  return v;
}

// Many rows (prefill): one CTA per row as in silu_mul_kernel, but silu(g) * u -- an exponential and a division
// per element -- is computed once and kept as packed bf16 (VPT x 16 bytes per thread) across the row-maximum
// reduction instead of being recomputed for the cast.  Same values, same bytes.
template <int VPT>
__global__ void __launch_bounds__(256) silu_mul_reg_kernel(const uint4* __restrict__ gate, const uint4* __restrict__ up,
                                                           int64_t ld_vec, int vec, uint4* __restrict__ h,
                                                           uint2* __restrict__ q, float* __restrict__ scale,
                                                           float* __restrict__ inv_scale,
                                                           unsigned int* __restrict__ group_amax, int64_t group_rows) {
  pdl_trigger();
  pdl_wait();
  const int64_t row = blockIdx.x;
  const uint4* gr = gate + row * ld_vec;
  const uint4* ur = up + row * ld_vec;
  uint4 hv[VPT];
  uint32_t m = 0;
#pragma unroll
  for (int k = 0; k < VPT; ++k) {
    const int i = threadIdx.x + k * 256;
    hv[k] = make_uint4(0, 0, 0, 0);
    if (i < vec) {
      float f[8];
      silu_mul8(__ldg(gr + i), __ldg(ur + i), f);
      hv[k] = pack8(f);
      if (h) h[row * vec + i] = hv[k];
#pragma unroll
      for (int j = 0; j < 8; ++j) m = max(m, mag_bits16(f[j]));
    }
  }
  const uint32_t row_bits = block_max_u32(m);
  if (group_amax && threadIdx.x == 0) atomicMax(group_amax + row / group_rows, row_bits << 16);
  if (!q) return;
  const float s = current_scale_from_amax(bf16_bits_to_float(row_bits));
#pragma unroll
  for (int k = 0; k < VPT; ++k) {
    const int i = threadIdx.x + k * 256;
    if (i < vec) q[row * vec + i] = quantize8_packed(hv[k], s);
  }
  if (threadIdx.x == 0) {
    scale[row] = s;
    inv_scale[row] = 1.0f / s;
  }
}

template <int VPT>
__global__ void __launch_bounds__(256) silu_mul_cluster_kernel(const uint4* __restrict__ gate,
                                                               const uint4* __restrict__ up, int64_t ld_vec, int vec,
                                                               int C, uint4* __restrict__ h, uint2* __restrict__ q,
                                                               float* __restrict__ scale,
                                                               float* __restrict__ inv_scale,
                                                               unsigned int* __restrict__ group_amax,
                                                               int64_t group_rows) {
  pdl_trigger();
  pdl_wait();
  __shared__ uint32_t cta_max;
  const int64_t row = blockIdx.y;
  const int part = blockIdx.x;  // == rank in the cluster (cluster spans grid x)
  const int per = (vec + C - 1) / C;
  const int i0 = part * per;
  const int i1 = min(vec, i0 + per);
  const uint4* gr = gate + row * ld_vec;
  const uint4* ur = up + row * ld_vec;
  float hv[VPT][8];
  uint32_t m = 0;
#pragma unroll
  for (int k = 0; k < VPT; ++k) {
    const int i = i0 + threadIdx.x + k * 256;
    if (i < i1) {
      silu_mul8(__ldg(gr + i), __ldg(ur + i), hv[k]);
      if (h) h[row * vec + i] = pack8(hv[k]);
#pragma unroll
      for (int j = 0; j < 8; ++j) m = max(m, mag_bits16(hv[k][j]));
    }
  }
  const uint32_t mine = block_max_u32(m);
  if (threadIdx.x == 0) cta_max = mine;
  // cluster barrier: every CTA's partial maximum is published
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
  uint32_t row_bits = 0;
  for (int c = 0; c < C; ++c) row_bits = max(row_bits, ld_dsmem_u32(smem_u32(&cta_max), (uint32_t)c));
  // second barrier: nobody leaves (and frees its shared memory) while a peer may still read it
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
  if (group_amax && part == 0 && threadIdx.x == 0) atomicMax(group_amax + row / group_rows, row_bits << 16);
  if (!q) return;
  const float s = current_scale_from_amax(bf16_bits_to_float(row_bits));
#pragma unroll
  for (int k = 0; k < VPT; ++k) {
    const int i = i0 + threadIdx.x + k * 256;
    if (i < i1) q[row * vec + i] = quantize8f(hv[k], s);
  }
  if (part == 0 && threadIdx.x == 0) {
    scale[row] = s;
    inv_scale[row] = 1.0f / s;
  }
}

// RoPE + cache append, one CTA per new token, 16-byte accesses: work item = (head, 8 consecutive
// pair indices); q and k heads are rotated, v heads copied.
__global__ void __launch_bounds__(256) kv_append_rope_vec_kernel(
    const uint4* __restrict__ qkv, int64_t ld_vec, int T, int Hq, int Hkv, int D, const int32_t* __restrict__ positions,
    const uint4* __restrict__ cos_t, const uint4* __restrict__ sin_t, int64_t table_len, uint4* __restrict__ q_rot,
    uint4* __restrict__ k_cache, uint4* __restrict__ v_cache, int64_t max_len, int store_rotated_k, int* d_status) {
  pdl_trigger();
  pdl_wait();
  const int64_t bt = blockIdx.x;
  const int b = (int)(bt / T), t = (int)(bt % T);
  const int64_t pos = (int64_t)positions[b] + t;
  if (pos >= max_len || pos >= table_len || pos < 0) {
    if (threadIdx.x == 0) atomicCAS(d_status, 0, XAXB_CACHE_OVERFLOW * 1000 + 41);
    return;
  }
  const int hv = D / 16;       // 16-byte chunks per half head
  const int dv = D / 8;        // 16-byte chunks per head
  const int heads = Hq + 2 * Hkv;
  const uint4* src_row = qkv + bt * ld_vec;
  for (int w = threadIdx.x; w < heads * hv; w += blockDim.x) {
    const int head = w / hv, c = w % hv;
    const uint4* src = src_row + (int64_t)head * dv;
    const uint4 a = __ldg(src + c), bb = __ldg(src + c + hv);
    uint4 o1 = a, o2 = bb;
    if (head < Hq + Hkv && (head < Hq || store_rotated_k)) {
      rope_rotate_pieces(a, bb, __ldg(cos_t + pos * hv + c), __ldg(sin_t + pos * hv + c), o1, o2);
    }
    uint4* dst;
    if (head < Hq)
      dst = q_rot + (bt * Hq + head) * dv;
    else if (head < Hq + Hkv)
      dst = k_cache + (((int64_t)b * max_len + pos) * Hkv + (head - Hq)) * dv;
    else
      dst = v_cache + (((int64_t)b * max_len + pos) * Hkv + (head - Hq - Hkv)) * dv;
    dst[c] = o1;
    dst[c + hv] = o2;
  }
}

// ---------------------------------------------------------------------------------------

__global__ void __launch_bounds__(256) embed_kernel(const int32_t* __restrict__ tokens, const uint4* __restrict__ table,
                                                    int64_t vocab, int64_t vec, uint4* __restrict__ x, int* d_status) {
  pdl_trigger();
  pdl_wait();
  const int64_t i = blockIdx.x;
  int64_t t = tokens[i];
  if (t < 0 || t >= vocab) {  // the reference's gather clamps; report and clamp
    if (threadIdx.x == 0) atomicCAS(d_status, 0, XAXB_BAD_ARGUMENT * 1000 + 31);
    t = t < 0 ? 0 : vocab - 1;
  }
  for (int64_t j = threadIdx.x; j < vec; j += blockDim.x) x[i * vec + j] = __ldg(table + t * vec + j);
}

// arg-max with jnp.argmax semantics: first index of the maximum, NaN counts as the maximum.
__device__ __forceinline__ bool better(float v, int i, float bv, int bi) {
  const bool vn = v != v, bn = bv != bv;
  if (vn != bn) return vn;
  if (vn) return i < bi;
  return v > bv || (v == bv && i < bi);
}

__global__ void __launch_bounds__(1024) argmax_kernel(const __nv_bfloat16* __restrict__ logits, int64_t vocab,
                                                      int64_t ld, int32_t* __restrict__ out,
                                                      float* __restrict__ max_out) {
  pdl_trigger();
  pdl_wait();
  const int64_t row = blockIdx.x;
  const __nv_bfloat16* lr = logits + row * ld;
  float bv = -INFINITY;
  int bi = 0x7FFFFFFF;
  const int64_t vec = ((reinterpret_cast<uintptr_t>(lr) & 15) == 0) ? vocab / 8 : 0;
  for (int64_t i = threadIdx.x; i < vec; i += blockDim.x) {
    float f[8];
    unpack8(__ldg(reinterpret_cast<const uint4*>(lr) + i), f);
#pragma unroll
    for (int j = 0; j < 8; ++j)
      if (better(f[j], (int)(i * 8 + j), bv, bi)) bv = f[j], bi = (int)(i * 8 + j);
  }
  for (int64_t i = vec * 8 + threadIdx.x; i < vocab; i += blockDim.x) {
    const float v = __bfloat162float(lr[i]);
    if (better(v, (int)i, bv, bi)) bv = v, bi = (int)i;
  }
  __shared__ float sv[32];
  __shared__ int si[32];
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (better(ov, oi, bv, bi)) bv = ov, bi = oi;
  }
  if ((threadIdx.x & 31) == 0) sv[threadIdx.x >> 5] = bv, si[threadIdx.x >> 5] = bi;
  __syncthreads();
  if (threadIdx.x < 32) {
    const int nw = (blockDim.x + 31) >> 5;
    bv = threadIdx.x < nw ? sv[threadIdx.x] : -INFINITY;
    bi = threadIdx.x < nw ? si[threadIdx.x] : 0x7FFFFFFF;
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (better(ov, oi, bv, bi)) bv = ov, bi = oi;
    }
    if (threadIdx.x == 0) {
      out[row] = bi;
      if (max_out) max_out[row] = bv;
    }
  }
}

// Vocabulary-sharded arg-max: part p holds (max value, local index) of vocabulary slice p for
// every row; the winner's global index is p * slice + local index.  Lower part wins ties, which
// is the lower global index.
__global__ void argmax_merge_kernel(const float* __restrict__ vals, const int32_t* __restrict__ idx, int parts,
                                    int rows, int slice, int32_t* __restrict__ out) {
  pdl_trigger();
  pdl_wait();
  const int r = blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= rows) return;
  float bv = vals[r];
  int bi = idx[r];
  for (int p = 1; p < parts; ++p) {
    const float v = vals[p * rows + r];
    const int i = p * slice + idx[p * rows + r];
    if (better(v, i, bv, bi)) bv = v, bi = i;
  }
  out[r] = bi;
}

// ---------------------------------------------------------------------------------------
// QK-norm (xax/arch/attention.py:864-867): RMSNorm over head_dim of every query and key head,
// in place on the fused projection output qkv [rows, (Hq + 2 Hkv) * D] (row stride ld), before
// RoPE.  One warp per (row, head); arithmetic and rounding are RMSNorm's (rmsnorm_kernel).
__global__ void __launch_bounds__(32) qk_norm_kernel(__nv_bfloat16* __restrict__ qkv, int64_t ld, int Hq, int Hkv, int D,
                                                     const __nv_bfloat16* __restrict__ wq,
                                                     const __nv_bfloat16* __restrict__ wk, float eps) {
  pdl_trigger();
  pdl_wait();
  const int64_t row = blockIdx.x;
  const int head = blockIdx.y;  // 0 .. Hq + Hkv - 1: query heads, then key heads
  const __nv_bfloat16* w = head < Hq ? wq : wk;
  if (!w) return;
  __nv_bfloat16* x = qkv + row * ld + (int64_t)head * D;
  float acc = 0.0f;
  for (int i = threadIdx.x; i < D; i += 32) {
    const float v = __bfloat162float(x[i]);
    acc += bf16_round(v * v);
  }
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  const float mean = bf16_round(acc / (float)D);
  const float n = bf16_round(sqrtf(bf16_round(mean + bf16_round(eps))));
  for (int i = threadIdx.x; i < D; i += 32) {
    const float v = __bfloat162float(x[i]);
    x[i] = __float2bfloat16_rn(bf16_round(v / n) * __bfloat162float(w[i]));
  }
}

// ---------------------------------------------------------------------------------------
// RoPE on its own (xax/arch/attention.py:443-526): x [rows, heads, D] bf16, row r at position
// positions[r].  Grid (rows, heads), D/2 threads; thread i owns pair i of the chosen style:
// "concatenated" pairs (i, i + D/2), "interleaved" pairs (2i, 2i + 1).  Every product and
// sum rounds to bf16, as the reference's bf16 arithmetic does.
__global__ void rope_apply_kernel(const __nv_bfloat16* __restrict__ x, int heads, int D,
                                  const int32_t* __restrict__ positions, const __nv_bfloat16* __restrict__ cos_t,
                                  const __nv_bfloat16* __restrict__ sin_t, int64_t table_len, int interleaved,
                                  __nv_bfloat16* __restrict__ out, int* d_status) {
  pdl_trigger();
  pdl_wait();
  const int64_t row = blockIdx.x;
  const int head = blockIdx.y, i = threadIdx.x, half = D / 2;
  const int64_t pos = positions[row];
  if (pos < 0 || pos >= table_len) {
    if (i == 0) atomicCAS(d_status, 0, XAXB_CACHE_OVERFLOW * 1000 + 45);
    return;
  }
  const int64_t base = (row * heads + head) * D;
  const int ia = interleaved ? 2 * i : i, ib = interleaved ? 2 * i + 1 : i + half;
  const float xa = __bfloat162float(x[base + ia]), xb = __bfloat162float(x[base + ib]);
  const float c = __bfloat162float(cos_t[pos * half + i]), s = __bfloat162float(sin_t[pos * half + i]);
  out[base + ia] = __float2bfloat16_rn(bf16_round(xa * c) - bf16_round(xb * s));
  out[base + ib] = interleaved ? __float2bfloat16_rn(bf16_round(xa * s) + bf16_round(xb * c))
                               : __float2bfloat16_rn(bf16_round(xb * c) + bf16_round(xa * s));
}

// ---------------------------------------------------------------------------------------
// RoPE ("concatenated" halves) + cache append.  Grid (B*T, Hq + 2*Hkv); D/2 threads: thread i
// owns the pair (i, i + D/2).  out1 = bf16(bf16(x1*c) - bf16(x2*s)), out2 = bf16(bf16(x2*c) + bf16(x1*s)).

__global__ void kv_append_rope_kernel(const __nv_bfloat16* __restrict__ qkv, int64_t ld, int T, int Hq, int Hkv, int D,
                                      const int32_t* __restrict__ positions, const __nv_bfloat16* __restrict__ cos_t,
                                      const __nv_bfloat16* __restrict__ sin_t, int64_t table_len,
                                      __nv_bfloat16* __restrict__ q_rot, __nv_bfloat16* __restrict__ k_cache,
                                      __nv_bfloat16* __restrict__ v_cache, int64_t max_len, int store_rotated_k,
                                      int* d_status) {
  pdl_trigger();
  pdl_wait();
  const int64_t bt = blockIdx.x;
  const int b = (int)(bt / T), t = (int)(bt % T);
  const int head = blockIdx.y;
  const int i = threadIdx.x, half = D / 2;
  const int64_t pos = (int64_t)positions[b] + t;
  if (pos >= max_len || pos >= table_len || pos < 0) {
    if (i == 0) atomicCAS(d_status, 0, XAXB_CACHE_OVERFLOW * 1000 + 41);
    return;
  }
  const __nv_bfloat16* src = qkv + bt * ld + (int64_t)head * D;
  const float x1 = __bfloat162float(src[i]), x2 = __bfloat162float(src[i + half]);
  const float c = __bfloat162float(cos_t[pos * half + i]), s = __bfloat162float(sin_t[pos * half + i]);
  const float r1 = bf16_round(bf16_round(x1 * c) - bf16_round(x2 * s));
  const float r2 = bf16_round(bf16_round(x2 * c) + bf16_round(x1 * s));
  if (head < Hq) {
    __nv_bfloat16* dst = q_rot + (bt * Hq + head) * D;
    dst[i] = __float2bfloat16_rn(r1);
    dst[i + half] = __float2bfloat16_rn(r2);
  } else if (head < Hq + Hkv) {
    __nv_bfloat16* dst = k_cache + (((int64_t)b * max_len + pos) * Hkv + (head - Hq)) * D;
    dst[i] = store_rotated_k ? __float2bfloat16_rn(r1) : src[i];
    dst[i + half] = store_rotated_k ? __float2bfloat16_rn(r2) : src[i + half];
  } else {
    __nv_bfloat16* dst = v_cache + (((int64_t)b * max_len + pos) * Hkv + (head - Hq - Hkv)) * D;
    dst[i] = src[i];
    dst[i + half] = src[i + half];
  }
}

__global__ void advance_positions_kernel(int32_t* positions, int B, int32_t delta) {
  pdl_trigger();
  pdl_wait();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < B) positions[i] += delta;
}

// ---------------------------------------------------------------------------------------
// Check kernels (CUDA cores, reference order of operations).

__global__ void gemm_fp8_check_kernel(const __nv_fp8_storage_t* __restrict__ a, int64_t lda,
                                      const __nv_fp8_storage_t* __restrict__ b, int64_t ldb, int64_t M, int64_t N,
                                      int64_t K, const float* row_mul, int rms, const float* col_mul, int cms,
                                      const __nv_bfloat16* bias, const __nv_bfloat16* residual, int64_t ldr,
                                      __nv_bfloat16* out, int64_t ldo) {
  pdl_trigger();
  pdl_wait();
  const int64_t n = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t m = blockIdx.y;
  if (n >= N || m >= M) return;
  float acc = 0.0f;
  for (int64_t k = 0; k < K; ++k) {
    const float av = __half2float(__half(__nv_cvt_fp8_to_halfraw(a[m * lda + k], __NV_E4M3)));
    const float bv = __half2float(__half(__nv_cvt_fp8_to_halfraw(b[n * ldb + k], __NV_E4M3)));
    acc = fmaf(av, bv, acc);
  }
  float v = acc * (row_mul ? row_mul[m * rms] : 1.0f) * (col_mul ? col_mul[n * cms] : 1.0f);
  if (bias) v += __bfloat162float(bias[n]);
  if (residual) v += __bfloat162float(residual[m * ldr + n]);
  out[m * ldo + n] = __float2bfloat16_rn(v);
}

// One CTA per (query, head): logits to shared memory, float32 softmax, probabilities
// rounded to bf16, P.V accumulated in float32.
__global__ void __launch_bounds__(128) attn_check_kernel(const __nv_bfloat16* __restrict__ q,
                                                         const __nv_bfloat16* __restrict__ kc,
                                                         const __nv_bfloat16* __restrict__ vc,
                                                         const int32_t* __restrict__ positions, int T, int Hq, int Hkv,
                                                         int D, int64_t max_len, float sm_scale,
                                                         __nv_bfloat16* __restrict__ out) {
  pdl_trigger();
  pdl_wait();
  extern __shared__ float logits[];
  __shared__ float red[4];
  const int h = blockIdx.x;
  const int64_t bt = blockIdx.y;
  const int b = (int)(bt / T), t = (int)(bt % T);
  const int g = h / (Hq / Hkv);
  const int L = positions[b] + t + 1;
  const __nv_bfloat16* qv = q + (bt * Hq + h) * D;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int j = warp; j < L; j += 4) {
    const __nv_bfloat16* kr = kc + (((int64_t)b * max_len + j) * Hkv + g) * D;
    float p = 0.0f;
    for (int d = lane; d < D; d += 32) p = fmaf(__bfloat162float(qv[d]), __bfloat162float(kr[d]), p);
    for (int o = 16; o > 0; o >>= 1) p += __shfl_xor_sync(0xffffffffu, p, o);
    if (lane == 0) logits[j] = p * sm_scale;
  }
  __syncthreads();
  float m = -INFINITY;
  for (int j = threadIdx.x; j < L; j += blockDim.x) m = fmaxf(m, logits[j]);
  for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  if (lane == 0) red[warp] = m;
  __syncthreads();
  m = fmaxf(fmaxf(red[0], red[1]), fmaxf(red[2], red[3]));
  __syncthreads();
  float sum = 0.0f;
  for (int j = threadIdx.x; j < L; j += blockDim.x) {
    const float e = expf(logits[j] - m);
    logits[j] = e;
    sum += e;
  }
  for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
  if (lane == 0) red[warp] = sum;
  __syncthreads();
  sum = red[0] + red[1] + red[2] + red[3];
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    float acc = 0.0f;
    for (int j = 0; j < L; ++j) {
      const float p = bf16_round(logits[j] / sum);
      acc = fmaf(p, __bfloat162float(vc[(((int64_t)b * max_len + j) * Hkv + g) * D + d]), acc);
    }
    out[(bt * Hq + h) * D + d] = __float2bfloat16_rn(acc);
  }
}

}  // namespace xaxb

using namespace xaxb;

static int row_threads(int64_t vec) {
  int t = (int)((vec + 31) / 32 * 32);
  return t > 256 ? 256 : (t < 32 ? 32 : t);
}

extern "C" {

int xaxb_rmsnorm(xaxb_ctx* ctx, void* stream, const void* x_bf16, const void* weight_bf16, float eps, int64_t rows,
                 int64_t dim, void* y_bf16, void* q_e4m3, float* scale, float* inv_scale, float* group_amax,
                 int64_t group_rows) {
  if (!ctx || !x_bf16 || !weight_bf16 || rows <= 0 || dim <= 0 || dim % 8 != 0) {
    set_last_error("rmsnorm: null pointer, or dim (%lld) not a positive multiple of 8", (long long)dim);
    return XAXB_BAD_ARGUMENT;
  }
  if (q_e4m3 && (!scale || !inv_scale)) return XAXB_BAD_ARGUMENT;
  if (group_amax && group_rows <= 0) return XAXB_BAD_ARGUMENT;
  if ((reinterpret_cast<uintptr_t>(x_bf16) | reinterpret_cast<uintptr_t>(weight_bf16) |
       reinterpret_cast<uintptr_t>(y_bf16)) & 15) {
    set_last_error("rmsnorm: pointers must be 16-byte aligned");
    return XAXB_BAD_ARGUMENT;
  }
  const int64_t vec = dim / 8;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const uint4* xp = static_cast<const uint4*>(x_bf16);
  const uint4* wp = static_cast<const uint4*>(weight_bf16);
  uint4* yp = static_cast<uint4*>(y_bf16);
  uint2* qp = static_cast<uint2*>(q_e4m3);
  unsigned int* gp = reinterpret_cast<unsigned int*>(group_amax);
  const int64_t gr = group_rows > 0 ? group_rows : 1;
  const bool few_rows = rows <= 2 * reinterpret_cast<const Ctx*>(ctx)->num_sms;
  if (few_rows && vec > 256 && vec <= 512)
    launch_kernel(rmsnorm_reg_kernel<1, 512>, dim3((unsigned)rows), dim3(512), 0, st, 1, xp, wp, eps, (int)vec, yp, qp, scale, inv_scale, gp, gr);
  else if (few_rows && vec > 512 && vec <= 1024)
    launch_kernel(rmsnorm_reg_kernel<1, 1024>, dim3((unsigned)rows), dim3(1024), 0, st, 1, xp, wp, eps, (int)vec, yp, qp, scale, inv_scale, gp, gr);
  // Many rows (prefill): a row's work is one dependent chain (load, sum, normalise, maximum, store), so what
  // counts is how many rows an SM has in flight: narrow CTAs with four 16-byte pieces per thread keep four times
  // as many rows and loads in flight as one piece per thread (4096 x 2048: 17 -> 9 us).
  else if (!few_rows && vec > 64 && vec <= 256)
    launch_kernel(rmsnorm_reg_kernel<4, 64>, dim3((unsigned)rows), dim3(64), 0, st, 1, xp, wp, eps, (int)vec, yp, qp, scale, inv_scale, gp, gr);
  else if (!few_rows && vec > 256 && vec <= 512)
    launch_kernel(rmsnorm_reg_kernel<4, 128>, dim3((unsigned)rows), dim3(128), 0, st, 1, xp, wp, eps, (int)vec, yp, qp, scale, inv_scale, gp, gr);
  else if (vec > 64 && vec <= 256)
    launch_kernel(rmsnorm_reg_kernel<1>, dim3((unsigned)rows), dim3(256), 0, st, 1, xp, wp, eps, (int)vec, yp, qp, scale, inv_scale, gp, gr);
  else if (vec > 256 && vec <= 512)
    launch_kernel(rmsnorm_reg_kernel<2>, dim3((unsigned)rows), dim3(256), 0, st, 1, xp, wp, eps, (int)vec, yp, qp, scale, inv_scale, gp, gr);
  else if (vec > 512 && vec <= 1024)
    launch_kernel(rmsnorm_reg_kernel<4>, dim3((unsigned)rows), dim3(256), 0, st, 1, xp, wp, eps, (int)vec, yp, qp, scale, inv_scale, gp, gr);
  else
    launch_kernel(rmsnorm_kernel, dim3((unsigned)rows), dim3(row_threads(vec)), 0, st, 1, xp, wp, eps, vec, yp, qp, scale, inv_scale, gp, gr);
  return check_launch("rmsnorm_kernel");
}

int xaxb_silu_mul(xaxb_ctx* ctx, void* stream, const void* gate_bf16, const void* up_bf16, int64_t ld, int64_t rows,
                  int64_t dim, void* h_bf16, void* q_e4m3, float* scale, float* inv_scale, float* group_amax,
                  int64_t group_rows) {
  if (!ctx || !gate_bf16 || rows <= 0 || dim <= 0 || dim % 8 != 0 || ld % 8 != 0) {
    set_last_error("silu_mul: null pointer, or dim/ld not positive multiples of 8");
    return XAXB_BAD_ARGUMENT;
  }
  if (q_e4m3 && (!scale || !inv_scale)) return XAXB_BAD_ARGUMENT;
  if (group_amax && group_rows <= 0) return XAXB_BAD_ARGUMENT;
  const uint4* gate = static_cast<const uint4*>(gate_bf16);
  const uint4* up = up_bf16 ? static_cast<const uint4*>(up_bf16) : gate + dim / 8;
  if ((reinterpret_cast<uintptr_t>(gate) | reinterpret_cast<uintptr_t>(up) | reinterpret_cast<uintptr_t>(h_bf16)) &
      15) {
    set_last_error("silu_mul: pointers must be 16-byte aligned");
    return XAXB_BAD_ARGUMENT;
  }
  const int64_t vec = dim / 8;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  uint4* hp = static_cast<uint4*>(h_bf16);
  uint2* qp = static_cast<uint2*>(q_e4m3);
  unsigned int* gp = reinterpret_cast<unsigned int*>(group_amax);
  const int64_t gr = group_rows > 0 ? group_rows : 1;
  // rows wide enough to be worth spreading, few enough rows that one CTA per row starves the GPU
  if (vec >= 256 && rows <= 65535 && rows < 2048) {
    int C = (int)((vec + 255) / 256);
    if (C > 8) C = 8;
    const int64_t per = (vec + C - 1) / C;
    const int vpt = (int)((per + 255) / 256);
    if (vpt <= 2) {
      const dim3 cgrid((unsigned)C, (unsigned)rows, 1);
      cudaError_t e;
      if (vpt == 1)
        e = launch_kernel(silu_mul_cluster_kernel<1>, cgrid, dim3(256), 0, st, (unsigned)C, gate, up, ld / 8, (int)vec, C,
                          hp, qp, scale, inv_scale, gp, gr);
      else
        e = launch_kernel(silu_mul_cluster_kernel<2>, cgrid, dim3(256), 0, st, (unsigned)C, gate, up, ld / 8, (int)vec, C,
                          hp, qp, scale, inv_scale, gp, gr);
      if (e != cudaSuccess) {
        set_last_error("silu_mul_cluster_kernel launch: %s", cudaGetErrorString(e));
        return XAXB_LAUNCH_FAILED;
      }
      return check_launch("silu_mul_cluster_kernel");
    }
  }
  if ((qp || gp) && vec > 256 && vec <= 8 * 256) {  // the row fits the registers of one 256-thread CTA
    const int vpt = (int)((vec + 255) / 256);
    const dim3 grid((unsigned)rows);
#define XAXB_SILU_REG(V)                                                                                        \
  launch_kernel(silu_mul_reg_kernel<V>, grid, dim3(256), 0, st, 1, gate, up, ld / 8, (int)vec, hp, qp, scale, \
                inv_scale, gp, gr)
    if (vpt <= 2) XAXB_SILU_REG(2);
    else if (vpt <= 3) XAXB_SILU_REG(3);
    else if (vpt <= 4) XAXB_SILU_REG(4);
    else if (vpt <= 6) XAXB_SILU_REG(6);
    else XAXB_SILU_REG(8);
#undef XAXB_SILU_REG
    return check_launch("silu_mul_reg_kernel");
  }
  launch_kernel(silu_mul_kernel, dim3((unsigned)rows), dim3(row_threads(vec)), 0, st, 1, gate, up, ld / 8, vec, hp, qp, scale, inv_scale, gp, gr,
                                                               TpRowMax{}, nullptr);
  return check_launch("silu_mul_kernel");
}

int xaxb_silu_mul_cast_tp(xaxb_ctx* ctx, void* stream, const void* gate_bf16, const void* up_bf16, int64_t ld,
                          int64_t rows, int64_t dim, void* q_e4m3, float* scale, float* inv_scale,
                          void* const* peer_bases, int rank, int world, int64_t inbox_offset_bytes,
                          int64_t sync_offset_bytes) {
  if (!ctx || !gate_bf16 || !q_e4m3 || !scale || !inv_scale || rows <= 0 || dim <= 0 || dim % 8 != 0 || ld % 8 != 0) {
    set_last_error("silu_mul_cast_tp: null pointer, or dim/ld not positive multiples of 8");
    return XAXB_BAD_ARGUMENT;
  }
  if (rows > kTpMaxSlots) {
    set_last_error("silu_mul_cast_tp: at most %d rows", kTpMaxSlots);
    return XAXB_UNSUPPORTED;
  }
  TpRowMax tp;
  int rc = fill_tp_rowmax(tp, peer_bases, rank, world, inbox_offset_bytes, sync_offset_bytes, "silu_mul_cast_tp");
  if (rc) return rc;
  const uint4* gate = static_cast<const uint4*>(gate_bf16);
  const uint4* up = up_bf16 ? static_cast<const uint4*>(up_bf16) : gate + dim / 8;
  if ((reinterpret_cast<uintptr_t>(gate) | reinterpret_cast<uintptr_t>(up)) & 15) {
    set_last_error("silu_mul_cast_tp: pointers must be 16-byte aligned");
    return XAXB_BAD_ARGUMENT;
  }
  const int64_t vec = dim / 8;
  // one CTA per token row (the row's amax is exchanged by the CTA as a whole); with at most 1024 rows a CTA
  // is alone on its SM or nearly so, and what bounds it is each thread's own instruction stream: one 16-byte
  // piece per thread where the row allows
  int threads = (int)((vec + 31) / 32 * 32);
  threads = threads < 256 ? 256 : (threads > 1024 ? 1024 : threads);
  launch_kernel(silu_mul_kernel, dim3((unsigned)rows), dim3((unsigned)threads), 0, static_cast<cudaStream_t>(stream), 1,
      gate, up, ld / 8, vec, nullptr, static_cast<uint2*>(q_e4m3), scale, inv_scale, nullptr, 1, tp,
      reinterpret_cast<Ctx*>(ctx)->d_status);
  return check_launch("silu_mul_kernel (tensor-parallel)");
}

int xaxb_embed(xaxb_ctx* ctx, void* stream, const int32_t* tokens, int64_t n_tokens, const void* table_bf16,
               int64_t vocab, int64_t dim, void* x_bf16) {
  if (!ctx || !tokens || !table_bf16 || !x_bf16 || n_tokens <= 0 || dim <= 0 || dim % 8 != 0 || vocab <= 0)
    return XAXB_BAD_ARGUMENT;
  Ctx* c = reinterpret_cast<Ctx*>(ctx);
  launch_kernel(embed_kernel, dim3((unsigned)n_tokens), dim3(row_threads(dim / 8)), 0, static_cast<cudaStream_t>(stream), 1, 
      tokens, static_cast<const uint4*>(table_bf16), vocab, dim / 8, static_cast<uint4*>(x_bf16), c->d_status);
  return check_launch("embed_kernel");
}

int xaxb_argmax(xaxb_ctx* ctx, void* stream, const void* logits_bf16, int64_t rows, int64_t vocab, int64_t ld,
                int32_t* out, float* max_out) {
  if (!ctx || !logits_bf16 || !out || rows <= 0 || vocab <= 0 || ld < vocab) return XAXB_BAD_ARGUMENT;
  launch_kernel(argmax_kernel, dim3((unsigned)rows), dim3(1024), 0, static_cast<cudaStream_t>(stream), 1, 
      static_cast<const __nv_bfloat16*>(logits_bf16), vocab, ld, out, max_out);
  return check_launch("argmax_kernel");
}

int xaxb_argmax_merge(xaxb_ctx* ctx, void* stream, const float* part_max, const int32_t* part_idx, int64_t parts,
                      int64_t rows, int64_t slice, int32_t* out) {
  if (!ctx || !part_max || !part_idx || !out || parts <= 0 || rows <= 0 || slice <= 0) return XAXB_BAD_ARGUMENT;
  launch_kernel(argmax_merge_kernel, dim3((unsigned)((rows + 127) / 128)), dim3(128), 0, static_cast<cudaStream_t>(stream), 1, 
      part_max, part_idx, (int)parts, (int)rows, (int)slice, out);
  return check_launch("argmax_merge_kernel");
}

int xaxb_kv_append_rope(xaxb_ctx* ctx, void* stream, const void* qkv_bf16, int64_t ld, int64_t B, int64_t T,
                        int64_t Hq, int64_t Hkv, int64_t D, const int32_t* positions, const void* cos_bf16,
                        const void* sin_bf16, int64_t table_len, void* q_rot_bf16, void* k_cache_bf16,
                        void* v_cache_bf16, int64_t max_len, int store_rotated_k) {
  if (!ctx || !qkv_bf16 || !positions || !cos_bf16 || !sin_bf16 || !q_rot_bf16 || !k_cache_bf16 || !v_cache_bf16 ||
      B <= 0 || T <= 0 || Hq <= 0 || Hkv <= 0 || max_len <= 0)
    return XAXB_BAD_ARGUMENT;
  if (D % 2 != 0 || D < 2 || D > 2048 || ld < (Hq + 2 * Hkv) * D) {
    set_last_error("kv_append_rope: head_dim %lld / ld %lld not supported", (long long)D, (long long)ld);
    return XAXB_UNSUPPORTED;
  }
  if (Hq + 2 * Hkv > 65535) return XAXB_UNSUPPORTED;
  Ctx* c = reinterpret_cast<Ctx*>(ctx);
  if (D % 16 == 0 && ld % 8 == 0 &&
      ((reinterpret_cast<uintptr_t>(qkv_bf16) | reinterpret_cast<uintptr_t>(cos_bf16) |
        reinterpret_cast<uintptr_t>(sin_bf16) | reinterpret_cast<uintptr_t>(q_rot_bf16) |
        reinterpret_cast<uintptr_t>(k_cache_bf16) | reinterpret_cast<uintptr_t>(v_cache_bf16)) & 15) == 0) {
    const int items = (int)((Hq + 2 * Hkv) * (D / 16));
    int threads = (items + 31) / 32 * 32;
    if (threads > 256) threads = 256;
    launch_kernel(kv_append_rope_vec_kernel, dim3((unsigned)(B * T)), dim3(threads), 0, static_cast<cudaStream_t>(stream), 1, 
        static_cast<const uint4*>(qkv_bf16), ld / 8, (int)T, (int)Hq, (int)Hkv, (int)D, positions,
        static_cast<const uint4*>(cos_bf16), static_cast<const uint4*>(sin_bf16), table_len,
        static_cast<uint4*>(q_rot_bf16), static_cast<uint4*>(k_cache_bf16), static_cast<uint4*>(v_cache_bf16), max_len,
        store_rotated_k, c->d_status);
    return check_launch("kv_append_rope_vec_kernel");
  }
  dim3 grid((unsigned)(B * T), (unsigned)(Hq + 2 * Hkv));
  launch_kernel(kv_append_rope_kernel, grid, dim3((unsigned)(D / 2)), 0, static_cast<cudaStream_t>(stream), 1, 
      static_cast<const __nv_bfloat16*>(qkv_bf16), ld, (int)T, (int)Hq, (int)Hkv, (int)D, positions,
      static_cast<const __nv_bfloat16*>(cos_bf16), static_cast<const __nv_bfloat16*>(sin_bf16), table_len,
      static_cast<__nv_bfloat16*>(q_rot_bf16), static_cast<__nv_bfloat16*>(k_cache_bf16),
      static_cast<__nv_bfloat16*>(v_cache_bf16), max_len, store_rotated_k, c->d_status);
  return check_launch("kv_append_rope_kernel");
}

int xaxb_qk_norm(xaxb_ctx* ctx, void* stream, void* qkv_bf16, int64_t ld, int64_t rows, int64_t Hq, int64_t Hkv,
                 int64_t D, const void* q_weight_bf16, const void* k_weight_bf16, float eps) {
  if (!ctx || !qkv_bf16 || rows <= 0 || Hq <= 0 || Hkv <= 0 || D <= 0 || ld < (Hq + 2 * Hkv) * D ||
      (!q_weight_bf16 && !k_weight_bf16))
    return XAXB_BAD_ARGUMENT;
  if (Hq + Hkv > 65535) return XAXB_UNSUPPORTED;
  dim3 grid((unsigned)rows, (unsigned)(Hq + Hkv));
  launch_kernel(qk_norm_kernel, grid, dim3(32), 0, static_cast<cudaStream_t>(stream), 1,
                static_cast<__nv_bfloat16*>(qkv_bf16), ld, (int)Hq, (int)Hkv, (int)D,
                static_cast<const __nv_bfloat16*>(q_weight_bf16), static_cast<const __nv_bfloat16*>(k_weight_bf16), eps);
  return check_launch("qk_norm_kernel");
}

int xaxb_rope_apply(xaxb_ctx* ctx, void* stream, const void* x_bf16, int64_t rows, int64_t heads, int64_t D,
                    const int32_t* positions, const void* cos_bf16, const void* sin_bf16, int64_t table_len,
                    int interleaved, void* out_bf16) {
  if (!ctx || !x_bf16 || !positions || !cos_bf16 || !sin_bf16 || !out_bf16 || rows <= 0 || heads <= 0 ||
      table_len <= 0)
    return XAXB_BAD_ARGUMENT;
  if (D % 2 != 0 || D < 2 || D > 2048 || heads > 65535) {
    set_last_error("rope_apply: head_dim %lld / heads %lld not supported", (long long)D, (long long)heads);
    return XAXB_UNSUPPORTED;
  }
  Ctx* c = reinterpret_cast<Ctx*>(ctx);
  dim3 grid((unsigned)rows, (unsigned)heads);
  launch_kernel(rope_apply_kernel, grid, dim3((unsigned)(D / 2)), 0, static_cast<cudaStream_t>(stream), 1,
                static_cast<const __nv_bfloat16*>(x_bf16), (int)heads, (int)D, positions,
                static_cast<const __nv_bfloat16*>(cos_bf16), static_cast<const __nv_bfloat16*>(sin_bf16), table_len,
                interleaved, static_cast<__nv_bfloat16*>(out_bf16), c->d_status);
  return check_launch("rope_apply_kernel");
}

int xaxb_advance_positions(xaxb_ctx* ctx, void* stream, int32_t* positions, int64_t B, int32_t delta) {
  if (!ctx || !positions || B <= 0) return XAXB_BAD_ARGUMENT;
  launch_kernel(advance_positions_kernel, dim3((unsigned)((B + 127) / 128)), dim3(128), 0, static_cast<cudaStream_t>(stream), 1, positions,
                                                                                                        (int)B, delta);
  return check_launch("advance_positions_kernel");
}

int xaxb_gemm_fp8_check(xaxb_ctx* ctx, void* stream, const void* a_e4m3, int64_t lda, const void* b_e4m3,
                        int64_t ldb, int64_t M, int64_t N, int64_t K, const float* row_mul, int row_mul_stride,
                        const float* col_mul, int col_mul_stride, const void* bias_bf16, const void* residual_bf16,
                        int64_t ldr, void* out_bf16, int64_t ldo) {
  if (!ctx || !a_e4m3 || !b_e4m3 || !out_bf16 || M <= 0 || N <= 0 || K <= 0 || M > 65535) return XAXB_BAD_ARGUMENT;
  dim3 grid((unsigned)((N + 127) / 128), (unsigned)M);
  launch_kernel(gemm_fp8_check_kernel, grid, dim3(128), 0, static_cast<cudaStream_t>(stream), 1, 
      static_cast<const __nv_fp8_storage_t*>(a_e4m3), lda, static_cast<const __nv_fp8_storage_t*>(b_e4m3), ldb, M, N,
      K, row_mul, row_mul_stride, col_mul, col_mul_stride, static_cast<const __nv_bfloat16*>(bias_bf16),
      static_cast<const __nv_bfloat16*>(residual_bf16), ldr, static_cast<__nv_bfloat16*>(out_bf16), ldo);
  return check_launch("gemm_fp8_check_kernel");
}

int xaxb_attn_check(xaxb_ctx* ctx, void* stream, const void* q_rot_bf16, const void* k_cache_bf16,
                    const void* v_cache_bf16, const int32_t* positions, int64_t B, int64_t T, int64_t Hq, int64_t Hkv,
                    int64_t D, int64_t max_len, float softmax_scale, void* out_bf16) {
  if (!ctx || !q_rot_bf16 || !k_cache_bf16 || !v_cache_bf16 || !positions || !out_bf16 || B <= 0 || T <= 0 ||
      Hq <= 0 || Hkv <= 0 || Hq % Hkv != 0 || B * T > 65535)
    return XAXB_BAD_ARGUMENT;
  const size_t smem = (size_t)max_len * sizeof(float);
  if (smem > 200 * 1024) {
    set_last_error("attn_check: max_len %lld too long for the check kernel", (long long)max_len);
    return XAXB_UNSUPPORTED;
  }
  cudaFuncSetAttribute(attn_check_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  dim3 grid((unsigned)Hq, (unsigned)(B * T));
  launch_kernel(attn_check_kernel, grid, dim3(128), smem, static_cast<cudaStream_t>(stream), 1, 
      static_cast<const __nv_bfloat16*>(q_rot_bf16), static_cast<const __nv_bfloat16*>(k_cache_bf16),
      static_cast<const __nv_bfloat16*>(v_cache_bf16), positions, (int)T, (int)Hq, (int)Hkv, (int)D, max_len,
      softmax_scale, static_cast<__nv_bfloat16*>(out_bf16));
  return check_launch("attn_check_kernel");
}

}  // extern "C"
