// Kernel 1: fused amax reduce, scale computation and e4m3 cast.
//
// Bandwidth kernels: 128-bit loads (8 bf16), 64-bit stores (8 e4m3), warp-shuffle
// reductions.  The arithmetic mirrors the reference's bf16 op sequence so the bytes match:
// the scale is a bf16 value, the product x * scale is rounded to bf16, clipped to +-448
// and only then converted to e4m3 (round to nearest even).
#include "common.cuh"
#include "quant_device.cuh"

namespace xaxb {

// ---- per-row current scaling: one CTA per row, the row is swept twice (the second sweep
// hits L1/L2), so HBM sees one read of x and one write of q. ------------------------------
__global__ void __launch_bounds__(256) quantize_rows_kernel(const uint4* __restrict__ x, int64_t vec_per_row,
                                                            uint2* __restrict__ q, float* __restrict__ scale,
                                                            float* __restrict__ inv_scale, float* __restrict__ amax) {
  pdl_trigger();
  pdl_wait();
  const int64_t row = blockIdx.x;
  const uint4* xr = x + row * vec_per_row;
  uint32_t m = 0;
  for (int64_t i = threadIdx.x; i < vec_per_row; i += blockDim.x) m = absmax_bits8(m, __ldg(xr + i));
  const uint32_t row_bits = block_max_u32(m);
  const float a = bf16_bits_to_float(row_bits);
  const float s = current_scale_from_amax(a);
  uint2* qr = q + row * vec_per_row;
  for (int64_t i = threadIdx.x; i < vec_per_row; i += blockDim.x) qr[i] = quantize8_packed(__ldg(xr + i), s);
  if (threadIdx.x == 0) {
    scale[row] = s;
    inv_scale[row] = 1.0f / s;
    amax[row] = a;
  }
}

// The same for rows of up to NT * VPT pieces of 16 bytes, kept in registers between the two sweeps.  Launched
// with narrow CTAs when there are many rows: a row is one dependent chain (load, maximum, cast, store), and an
// SM overlaps as many chains as it has CTAs resident.
template <int VPT, int NT>
__global__ void __launch_bounds__(NT) quantize_rows_reg_kernel(const uint4* __restrict__ x, int vec_per_row,
                                                               uint2* __restrict__ q, float* __restrict__ scale,
                                                               float* __restrict__ inv_scale,
                                                               float* __restrict__ amax) {
  pdl_trigger();
  pdl_wait();
  const int64_t row = blockIdx.x;
  const uint4* xr = x + row * vec_per_row;
  uint4 v[VPT];
  uint32_t m = 0;
#pragma unroll
  for (int k = 0; k < VPT; ++k) {
    const int i = threadIdx.x + k * NT;
    v[k] = i < vec_per_row ? __ldg(xr + i) : make_uint4(0, 0, 0, 0);
  }
#pragma unroll
  for (int k = 0; k < VPT; ++k) m = absmax_bits8(m, v[k]);
  const uint32_t row_bits = block_max_u32(m);
  const float a = bf16_bits_to_float(row_bits);
  const float s = current_scale_from_amax(a);
  uint2* qr = q + row * vec_per_row;
#pragma unroll
  for (int k = 0; k < VPT; ++k) {
    const int i = threadIdx.x + k * NT;
    if (i < vec_per_row) qr[i] = quantize8_packed(v[k], s);
  }
  if (threadIdx.x == 0) {
    scale[row] = s;
    inv_scale[row] = 1.0f / s;
    amax[row] = a;
  }
}

// ---- per-group current scaling, pass 1: amax of each group of rows -------------------------
__global__ void __launch_bounds__(256) group_amax_kernel(const uint4* __restrict__ x, int64_t vec_per_group,
                                                         unsigned int* __restrict__ amax_bits) {
  pdl_trigger();
  pdl_wait();
  const int64_t g = blockIdx.y;
  const uint4* xg = x + g * vec_per_group;
  uint32_t m = 0;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < vec_per_group;
       i += (int64_t)gridDim.x * blockDim.x)
    m = absmax_bits8(m, __ldg(xg + i));
  const uint32_t r = block_max_u32(m);
  // bf16 magnitude bits widened to float bits: order-preserving, NaN stays the largest.
  if (threadIdx.x == 0) atomicMax(amax_bits + g, r << 16);
}

// ---- pass 2: scale from the group amax, cast ------------------------------------------------
__global__ void __launch_bounds__(256) group_cast_kernel(const uint4* __restrict__ x, int64_t vec_per_group,
                                                         int64_t group_rows, const float* __restrict__ amax,
                                                         uint2* __restrict__ q, float* __restrict__ scale,
                                                         float* __restrict__ inv_scale) {
  pdl_trigger();
  pdl_wait();
  const int64_t g = blockIdx.y;
  const float s = current_scale_from_amax(amax[g]);
  const uint4* xg = x + g * vec_per_group;
  uint2* qg = q + g * vec_per_group;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < vec_per_group;
       i += (int64_t)gridDim.x * blockDim.x)
    qg[i] = quantize8_packed(__ldg(xg + i), s);
  if (blockIdx.x == 0) {
    for (int64_t r = threadIdx.x; r < group_rows; r += blockDim.x) {
      scale[g * group_rows + r] = s;
      inv_scale[g * group_rows + r] = 1.0f / s;
    }
  }
}

__device__ __forceinline__ float nan_max(float a, float b) { return (a != a) ? a : ((b != b) ? b : fmaxf(a, b)); }

// ---- delayed scaling: cast with the incoming scale while reducing max|x|; the CTA that finishes
// last then produces the state for the next call:
//   history_out = roll(history_in, -1) with slot 0 <- amax; scale_out from max(history_out).
// One launch of 256-thread CTAs.  Four 16-byte loads are issued per thread before any is used, so a
// CTA keeps 16 KiB in flight.  scratch[0] collects max|x| (bf16 bits << 16), scratch[1] counts finished CTAs; both
// are zero on entry and the last CTA leaves them zero.  The history is staged in shared memory,
// so history_in and history_out may alias; scale_out may alias scale_in (every CTA has read it
// before the last one can finish).
__global__ void __launch_bounds__(256, 8) delayed_cast_kernel(const uint4* __restrict__ x, int64_t n_vec,
                                                           const float* scale_in, uint2* __restrict__ q,
                                                           unsigned int* scratch, const float* history_in,
                                                           int history_len, float* history_out, float* scale_out,
                                                           float* inv_scale_out) {
  pdl_trigger();
  pdl_wait();
  extern __shared__ float hist[];
  __shared__ float warp_max[8];
  __shared__ int is_last;
  const float old = *scale_in;
  const float s = bf16_round(old);
  uint32_t m = 0;
  // A CTA takes whole blocks of 4 x 256 vectors (16 KiB of x, contiguous), block index
  // blockIdx.x, blockIdx.x + gridDim.x, ...: thread t issues its four loads -- all of them, a
  // ragged last block included, under a predicate -- before it uses any of them.
  const int64_t n_blocks = (n_vec + 1023) / 1024;
  for (int64_t blk = blockIdx.x; blk < n_blocks; blk += gridDim.x) {
    const int64_t i0 = blk * 1024 + threadIdx.x;
    uint4 v[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const int64_t i = i0 + k * 256;
      v[k] = i < n_vec ? __ldg(x + i) : make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const int64_t i = i0 + k * 256;
      m = absmax_bits8(m, v[k]);
      if (q && i < n_vec) q[i] = quantize8_packed(v[k], s);
    }
  }
  const uint32_t r = block_max_u32(m);
  if (threadIdx.x == 0) {
    atomicMax(scratch, r << 16);
    __threadfence();
    is_last = atomicAdd(scratch + 1, 1u) == gridDim.x - 1;
  }
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  const float amax = __uint_as_float(atomicOr(scratch, 0u));
  for (int j = threadIdx.x; j < history_len; j += blockDim.x) {
    const int src = (j + 1 == history_len) ? 0 : j + 1;
    hist[j] = (j == 0) ? amax : history_in[src];
  }
  __syncthreads();
  float hm = -INFINITY;
  for (int j = threadIdx.x; j < history_len; j += blockDim.x) {
    history_out[j] = hist[j];
    hm = nan_max(hm, hist[j]);
  }
  for (int o = 16; o > 0; o >>= 1) hm = nan_max(hm, __shfl_xor_sync(0xffffffffu, hm, o));
  if ((threadIdx.x & 31) == 0) warp_max[threadIdx.x >> 5] = hm;
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < (int)(blockDim.x >> 5); ++w) hm = nan_max(hm, warp_max[w]);
    float sf = 448.0f / hm;  // float32: the bf16 constant promotes against the float32 history
    sf = (hm > 0.0f) ? sf : old;
    sf = isfinite(hm) ? sf : old;
    *scale_out = sf;
    if (inv_scale_out) *inv_scale_out = 1.0f / s;
    scratch[0] = 0u;
    scratch[1] = 0u;
  }
}

// ---- dequantise (xax/nn/fp8.py:123-138): out = compute_dtype(q) / compute_dtype(scale), one scale per
// row (stride 1) or one for the tensor (stride 0).  bf16: the quotient of the exact float32 images rounded to
// bf16, which is what a bf16 division yields; float32: a float32 division.  8 values per thread.
template <bool OUT_BF16>
__global__ void __launch_bounds__(256) dequantize_kernel(const uint2* __restrict__ q, int64_t vec_per_row,
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
      const __nv_fp8_storage_t byte = (__nv_fp8_storage_t)((w[k >> 2] >> ((k & 3) * 8)) & 0xFFu);
      const __half_raw h = __nv_cvt_fp8_to_halfraw(byte, __NV_E4M3);  // exact: every e4m3 value is a half
      f[k] = __half2float(__half(h)) / s;
    }
    if (OUT_BF16) {
      reinterpret_cast<uint4*>(out)[i] = pack8(f);
    } else {
      reinterpret_cast<float4*>(out)[2 * i] = make_float4(f[0], f[1], f[2], f[3]);
      reinterpret_cast<float4*>(out)[2 * i + 1] = make_float4(f[4], f[5], f[6], f[7]);
    }
  }
}

static int grid_for(int64_t n_vec, int num_sms, int64_t cap_per_group = 0) {
  int64_t blocks = (n_vec + 255) / 256;
  int64_t limit = cap_per_group > 0 ? cap_per_group : (int64_t)num_sms * 8;
  if (blocks > limit) blocks = limit;
  if (blocks < 1) blocks = 1;
  return (int)blocks;
}

}  // namespace xaxb

using namespace xaxb;

static int check_quant_args(const void* x, int64_t rows, int64_t cols) {
  if (!x || rows <= 0 || cols <= 0) {
    set_last_error("quantize: null input or non-positive shape (%lld x %lld)", (long long)rows, (long long)cols);
    return XAXB_BAD_ARGUMENT;
  }
  if (cols % 8 != 0 || (reinterpret_cast<uintptr_t>(x) & 15)) {
    set_last_error("quantize: cols (%lld) must be a multiple of 8 and x 16-byte aligned", (long long)cols);
    return XAXB_BAD_ARGUMENT;
  }
  return XAXB_OK;
}

extern "C" {

int xaxb_quantize_current(xaxb_ctx* ctx, void* stream, const void* x_bf16, int64_t rows, int64_t cols,
                          int64_t group_rows, void* q_e4m3, float* scale, float* inv_scale, float* amax) {
  if (!ctx || !q_e4m3 || !scale || !inv_scale || !amax) return XAXB_BAD_ARGUMENT;
  int rc = check_quant_args(x_bf16, rows, cols);
  if (rc) return rc;
  if (group_rows <= 0 || rows % group_rows != 0 || (reinterpret_cast<uintptr_t>(q_e4m3) & 7)) {
    set_last_error("quantize_current: rows (%lld) must be a multiple of group_rows (%lld), q 8-byte aligned",
                   (long long)rows, (long long)group_rows);
    return XAXB_BAD_ARGUMENT;
  }
  const Ctx* c = reinterpret_cast<const Ctx*>(ctx);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const uint4* x = static_cast<const uint4*>(x_bf16);
  uint2* q = static_cast<uint2*>(q_e4m3);
  if (group_rows == 1) {
    const int64_t vec = cols / 8;
    int threads = (int)((vec + 31) / 32 * 32);
    if (threads > 256) threads = 256;
    if (rows > 2 * c->num_sms && vec > 64 && vec <= 256)
      launch_kernel(quantize_rows_reg_kernel<4, 64>, dim3((unsigned)rows), dim3(64), 0, s, 1, x, (int)vec, q, scale, inv_scale, amax);
    else if (rows > 2 * c->num_sms && vec > 256 && vec <= 512)
      launch_kernel(quantize_rows_reg_kernel<4, 128>, dim3((unsigned)rows), dim3(128), 0, s, 1, x, (int)vec, q, scale, inv_scale, amax);
    else if (rows > 2 * c->num_sms && vec > 512 && vec <= 1024)
      launch_kernel(quantize_rows_reg_kernel<4, 256>, dim3((unsigned)rows), dim3(256), 0, s, 1, x, (int)vec, q, scale, inv_scale, amax);
    else
      launch_kernel(quantize_rows_kernel, dim3((unsigned)rows), dim3(threads), 0, s, 1, x, vec, q, scale, inv_scale, amax);
    return check_launch("quantize_rows_kernel");
  }
  const int64_t groups = rows / group_rows;
  const int64_t vec_per_group = group_rows * cols / 8;
  if (groups > 65535) {
    set_last_error("quantize_current: more than 65535 multi-row groups");
    return XAXB_UNSUPPORTED;
  }
  cudaMemsetAsync(amax, 0, groups * sizeof(float), s);
  int64_t cap = ((int64_t)c->num_sms * 8 + groups - 1) / groups;
  dim3 grid(grid_for(vec_per_group, c->num_sms, cap), (unsigned)groups);
  launch_kernel(group_amax_kernel, grid, dim3(256), 0, s, 1, x, vec_per_group, reinterpret_cast<unsigned int*>(amax));
  rc = check_launch("group_amax_kernel");
  if (rc) return rc;
  launch_kernel(group_cast_kernel, grid, dim3(256), 0, s, 1, x, vec_per_group, group_rows, amax, q, scale, inv_scale);
  return check_launch("group_cast_kernel");
}

int xaxb_group_amax(xaxb_ctx* ctx, void* stream, const void* x_bf16, int64_t rows, int64_t cols, int64_t group_rows,
                    float* amax) {
  if (!ctx || !amax) return XAXB_BAD_ARGUMENT;
  int rc = check_quant_args(x_bf16, rows, cols);
  if (rc) return rc;
  if (group_rows <= 0 || rows % group_rows != 0 || rows / group_rows > 65535) {
    set_last_error("group_amax: bad grouping rows=%lld group_rows=%lld", (long long)rows, (long long)group_rows);
    return XAXB_BAD_ARGUMENT;
  }
  const Ctx* c = reinterpret_cast<const Ctx*>(ctx);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int64_t groups = rows / group_rows;
  const int64_t vec_per_group = group_rows * cols / 8;
  cudaMemsetAsync(amax, 0, groups * sizeof(float), s);
  int64_t cap = ((int64_t)c->num_sms * 8 + groups - 1) / groups;
  dim3 grid(grid_for(vec_per_group, c->num_sms, cap), (unsigned)groups);
  launch_kernel(group_amax_kernel, grid, dim3(256), 0, s, 1, static_cast<const uint4*>(x_bf16), vec_per_group,
                                         reinterpret_cast<unsigned int*>(amax));
  return check_launch("group_amax_kernel");
}

int xaxb_quantize_with_amax(xaxb_ctx* ctx, void* stream, const void* x_bf16, int64_t rows, int64_t cols,
                            int64_t group_rows, const float* group_amax, void* q_e4m3, float* scale,
                            float* inv_scale) {
  if (!ctx || !q_e4m3 || !scale || !inv_scale || !group_amax) return XAXB_BAD_ARGUMENT;
  int rc = check_quant_args(x_bf16, rows, cols);
  if (rc) return rc;
  if (group_rows <= 0 || rows % group_rows != 0 || rows / group_rows > 65535) {
    set_last_error("quantize_with_amax: bad grouping rows=%lld group_rows=%lld", (long long)rows,
                   (long long)group_rows);
    return XAXB_BAD_ARGUMENT;
  }
  const Ctx* c = reinterpret_cast<const Ctx*>(ctx);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int64_t groups = rows / group_rows;
  const int64_t vec_per_group = group_rows * cols / 8;
  int64_t cap = ((int64_t)c->num_sms * 8 + groups - 1) / groups;
  dim3 grid(grid_for(vec_per_group, c->num_sms, cap), (unsigned)groups);
  launch_kernel(group_cast_kernel, grid, dim3(256), 0, s, 1, static_cast<const uint4*>(x_bf16), vec_per_group, group_rows, group_amax,
                                         static_cast<uint2*>(q_e4m3), scale, inv_scale);
  return check_launch("group_cast_kernel");
}

int xaxb_dequantize(xaxb_ctx* ctx, void* stream, const void* q_e4m3, int64_t rows, int64_t cols, const float* scale,
                    int scale_stride, int out_is_bf16, void* out) {
  if (!ctx || !q_e4m3 || !scale || !out || rows <= 0 || cols <= 0 || cols % 8 != 0 ||
      (scale_stride != 0 && scale_stride != 1) || (reinterpret_cast<uintptr_t>(q_e4m3) & 7) ||
      (reinterpret_cast<uintptr_t>(out) & 15)) {
    set_last_error("dequantize: null pointer, cols (%lld) not a multiple of 8, scale stride not 0 / 1, or misaligned "
                   "pointer", (long long)cols);
    return XAXB_BAD_ARGUMENT;
  }
  const Ctx* c = reinterpret_cast<const Ctx*>(ctx);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int64_t n_vec = rows * cols / 8;
  const dim3 grid(grid_for(n_vec, c->num_sms));
  if (out_is_bf16)
    launch_kernel(dequantize_kernel<true>, grid, dim3(256), 0, s, 1, static_cast<const uint2*>(q_e4m3), cols / 8, n_vec,
                  scale, scale_stride, out);
  else
    launch_kernel(dequantize_kernel<false>, grid, dim3(256), 0, s, 1, static_cast<const uint2*>(q_e4m3), cols / 8, n_vec,
                  scale, scale_stride, out);
  return check_launch("dequantize_kernel");
}

int xaxb_quantize_delayed(xaxb_ctx* ctx, void* stream, const void* x_bf16, int64_t rows, int64_t cols,
                          const float* scale_in, const float* history_in, int history_len, void* q_e4m3,
                          float* history_out, float* scale_out, float* inv_scale_out, float* amax_scratch) {
  if (!ctx || !scale_in || !history_in || !history_out || !scale_out || !amax_scratch) return XAXB_BAD_ARGUMENT;
  int rc = check_quant_args(x_bf16, rows, cols);
  if (rc) return rc;
  if (history_len <= 0 || history_len > 8192) {
    set_last_error("quantize_delayed: history_len %d outside [1, 8192]", history_len);
    return XAXB_BAD_ARGUMENT;
  }
  const Ctx* c = reinterpret_cast<const Ctx*>(ctx);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int64_t n_vec = rows * cols / 8;
  // one CTA per 16 KiB block of x while that fits one resident wave (8 CTAs per SM); beyond it the
  // CTAs loop.  Fewer CTAs also mean fewer arrivals at the ticket that elects the last one.
  int64_t grid = (n_vec + 1023) / 1024;
  if (grid > (int64_t)c->num_sms * 8) grid = (int64_t)c->num_sms * 8;
  launch_kernel(delayed_cast_kernel, dim3((unsigned)grid), dim3(256), history_len * sizeof(float), s, 1, 
      static_cast<const uint4*>(x_bf16), n_vec, scale_in, static_cast<uint2*>(q_e4m3),
      reinterpret_cast<unsigned int*>(amax_scratch), history_in, history_len, history_out, scale_out, inv_scale_out);
  return check_launch("delayed_cast_kernel");
}

}  // extern "C"
