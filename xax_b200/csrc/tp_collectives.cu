// Tensor-parallel exchange steps of the decode path over NVLink peer memory.
//
// Every rank owns one "symmetric" buffer (same size and layout on every rank) that all ranks of
// the box have mapped; a kernel gets the table of those mappings.  Two exchanges are needed per
// transformer block (xax/arch/llm.py:931-975: o_proj and down are row-parallel):
//
//   sum   the [tokens, hidden] bf16 partial outputs of a row-parallel projection.  The GEMM
//         writes its partial output straight into this rank's symmetric buffer; one CTA per
//         token row then waits until every rank's row is ready, reads the row from every rank
//         (plain peer loads, 16 bytes per thread), adds in float32 in rank order -- so every rank
//         computes the same bits -- and writes the bf16 row to local memory.
//   max   the per-token amax (float32 [tokens]) of the input of a row-parallel FP8 projection,
//         which spans all ranks.  Every rank stores its vector into every rank's inbox, raises a
//         flag there, waits for the others' flags and takes the maximum of its inbox.
//
// Readiness is signalled through 32-bit epoch counters in the symmetric buffer: slot (row, src)
// on rank dst holds the number of the last exchange whose data from `src` may be read by `dst`.
// Epochs only grow, every rank runs the same sequence of exchanges, and the local copy of the
// current epoch lives next to the flags, so a captured CUDA graph can be replayed.  All waits are
// bounded (the limit of every device-side wait in this library); a wait that gives up records
// XAXB_DEVICE_TIMEOUT with its site in the context's status word and the kernel carries on to its
// end with whatever it has -- nothing spins for ever and nothing traps.
//
// Data buffers are reused by the caller in alternation (two per exchange kind): a rank can only
// pass the flag wait of exchange k+1 after every other rank has finished reading exchange k, so
// the buffer of exchange k is free again at exchange k+2.  The max inbox alternates by epoch
// parity inside the kernel for the same reason.
//
// These kernels wait for kernels on OTHER GPUs.  They must never be launched as several ranks on
// one GPU: nothing guarantees that two such launches run at the same time.
#include "common.cuh"
#include "quant_device.cuh"
#include "tp_device.cuh"

namespace xaxb {

// One CTA per token row.  data_off: where every rank's [rows, cols] bf16 partial output starts
// in its symmetric buffer.
__global__ void __launch_bounds__(256) tp_allreduce_sum_kernel(const PeerTable peers, int64_t data_off,
                                                               int64_t sync_off, int rank, int world, int cols,
                                                               uint4* __restrict__ out, int* d_status) {
  pdl_trigger();
  pdl_wait();
  __shared__ uint32_t s_epoch;
  const int row = blockIdx.x;
  tp_exchange_flags(peers, sync_off, rank, world, row, &s_epoch, d_status, kSiteTpSum);
  const int vec = cols / 8;
  const int64_t row_off = data_off + (int64_t)row * cols * 2;
  for (int c = threadIdx.x; c < vec; c += blockDim.x) {
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    uint4 v[kTpMaxWorld];
#pragma unroll
    for (int r = 0; r < kTpMaxWorld; ++r)
      if (r < world) v[r] = ld_relaxed_sys_v4(peers.base[r] + row_off + (int64_t)c * 16);
#pragma unroll
    for (int r = 0; r < kTpMaxWorld; ++r) {
      if (r < world) {
        const uint32_t w[4] = {v[r].x, v[r].y, v[r].z, v[r].w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          acc[2 * j] += bf16_bits_to_float(w[j] & 0xFFFFu);
          acc[2 * j + 1] += bf16_bits_to_float(w[j] >> 16);
        }
      }
    }
    uint4 o;
    uint32_t* ow = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const uint32_t lo = __bfloat16_as_ushort(__float2bfloat16_rn(acc[2 * j]));
      const uint32_t hi = __bfloat16_as_ushort(__float2bfloat16_rn(acc[2 * j + 1]));
      ow[j] = lo | (hi << 16);
    }
    out[(int64_t)row * vec + c] = o;
  }
}

// The same exchange with the RMSNorm and per-token e4m3 cast that follow it in the block
// (xax/arch/attention.py:1487-1510: x + attn(..) feeds mlp_norm, x + ffn(..) feeds the next
// block's attn_norm) done on the summed row while it is still in registers: x (bf16) goes to
// local memory for the residual path, the normalised row only as e4m3 bytes and its scale.
// Arithmetic and rounding are those of rmsnorm_reg_kernel, so the bytes equal the unfused path's.
template <int VPT, int NT = 256>
__global__ void __launch_bounds__(NT) tp_allreduce_sum_norm_kernel(
    const PeerTable peers, int64_t data_off, int64_t sync_off, int rank, int world, int vec, uint4* __restrict__ x_out,
    const uint4* __restrict__ w, float eps, uint2* __restrict__ q, float* __restrict__ scale,
    float* __restrict__ inv_scale, int* d_status) {
  pdl_trigger();
  pdl_wait();
  __shared__ uint32_t s_epoch;
  const int64_t row = blockIdx.x;
  tp_exchange_flags(peers, sync_off, rank, world, (int)row, &s_epoch, d_status, kSiteTpSum);
  const int64_t row_off = data_off + row * vec * 16;
  float v[VPT][8];
  float acc = 0.0f;
#pragma unroll
  for (int k = 0; k < VPT; ++k) {
    const int i = threadIdx.x + k * NT;
    if (i < vec) {
      uint4 part[kTpMaxWorld];
#pragma unroll
      for (int r = 0; r < kTpMaxWorld; ++r)
        if (r < world) part[r] = ld_relaxed_sys_v4(peers.base[r] + row_off + (int64_t)i * 16);
      float s[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#pragma unroll
      for (int r = 0; r < kTpMaxWorld; ++r) {
        if (r < world) {
          float f[8];
          unpack8(part[r], f);
#pragma unroll
          for (int j = 0; j < 8; ++j) s[j] += f[j];
        }
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        v[k][j] = bf16_round(s[j]);
        acc += bf16_round(v[k][j] * v[k][j]);
      }
      x_out[row * vec + i] = pack8(v[k]);
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
    }
  }
  const uint32_t row_bits = block_max_u32(m);
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

// ---- push variant of the sum -----------------------------------------------------------------
// The row-parallel GEMM itself writes its bf16 partial output into slot `rank` of EVERY rank's
// staging buffer ([world][rows][cols]) from its epilogue and adds the number of 16-byte pieces it
// completed to an arrival counter on every rank (xaxb_gemm_fp8_push).  The consumer below waits
// until the local counter has reached the running total expected so far -- world x rows x cols / 8
// pieces per exchange -- and then reads LOCAL memory only: no flag raising, no trip over NVLink on
// its critical path.  Staging buffer and counter come in pairs used in alternation, so that pieces of
// exchange k+1 can never be taken for pieces of exchange k.  The running totals live in local
// memory (one per token row and counter), so a captured step can be replayed.
constexpr int kSiteTpPush = 46;

template <int VPT, int NT = 256>
__global__ void __launch_bounds__(NT) tp_push_sum_norm_kernel(
    const uint8_t* __restrict__ staging, int64_t slot_stride, const unsigned int* counter, unsigned int* totals,
    unsigned int pieces_per_exchange, int world, int vec, uint4* __restrict__ x_out, const uint4* __restrict__ w,
    float eps, uint2* __restrict__ q, float* __restrict__ scale, float* __restrict__ inv_scale, int* d_status) {
  pdl_trigger();
  pdl_wait();
  const int64_t row = blockIdx.x;
  if (threadIdx.x == 0) {
    const unsigned int want = totals[row] + pieces_per_exchange;
    totals[row] = want;
    if ((int32_t)(ld_acquire_sys(counter) - want) < 0) {
      const unsigned long long t0 = globaltimer_ns();
      const unsigned long long limit = peer_wait_limit_ns(d_status);
      while ((int32_t)(ld_acquire_sys(counter) - want) < 0) {
        __nanosleep(32);  // a hundred CTAs poll at once: leave the memory system to the stores they wait for
        if (*reinterpret_cast<volatile int*>(d_status) != 0) break;
        if (globaltimer_ns() - t0 > limit) {
          atomicCAS(d_status, 0, XAXB_DEVICE_TIMEOUT * 1000 + kSiteTpPush);
          break;
        }
      }
    }
  }
  __syncthreads();
  const int64_t row_off = row * vec * 16;
  float v[VPT][8];
  float acc = 0.0f;
#pragma unroll
  for (int k = 0; k < VPT; ++k) {
    const int i = threadIdx.x + k * NT;
    if (i < vec) {
      uint4 part[kTpMaxWorld];
#pragma unroll
      for (int r = 0; r < kTpMaxWorld; ++r)
        if (r < world) part[r] = ld_relaxed_sys_v4(staging + r * slot_stride + row_off + (int64_t)i * 16);
      float s[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#pragma unroll
      for (int r = 0; r < kTpMaxWorld; ++r) {
        if (r < world) {
          float f[8];
          unpack8(part[r], f);
#pragma unroll
          for (int j = 0; j < 8; ++j) s[j] += f[j];
        }
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        v[k][j] = bf16_round(s[j]);
        acc += bf16_round(v[k][j] * v[k][j]);
      }
      x_out[row * vec + i] = pack8(v[k]);
    }
  }
  if (!w) return;  // plain sum: no norm, no cast (uniform over the CTA)
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
    }
  }
  const uint32_t row_bits = block_max_u32(m);
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

// One CTA; n <= 1024 values.  inbox_off: float32 [2][kTpMaxWorld][kTpMaxSlots] in the symmetric
// buffer (two copies, used in alternation by epoch parity).
__global__ void __launch_bounds__(1024) tp_allreduce_max_kernel(const PeerTable peers, int64_t inbox_off,
                                                                int64_t sync_off, int rank, int world, int n,
                                                                const float* __restrict__ in, float* __restrict__ out,
                                                                int* d_status) {
  pdl_trigger();
  pdl_wait();
  __shared__ uint32_t s_epoch;
  const int i = threadIdx.x;
  // the epoch this exchange will get decides which inbox copy it uses
  const uint32_t* my_epoch =
      reinterpret_cast<const uint32_t*>(peers.base[rank] + sync_off) + kTpMaxSlots * kTpMaxWorld;
  const uint32_t parity = (*my_epoch + 1) & 1;
  const int64_t box = inbox_off + (int64_t)parity * kTpMaxWorld * kTpMaxSlots * 4;
  const float mine = i < n ? in[i] : 0.0f;
  if (i < n) {
#pragma unroll
    for (int r = 0; r < kTpMaxWorld; ++r)
      if (r < world)
        st_relaxed_sys_f32(reinterpret_cast<float*>(peers.base[r] + box) + rank * kTpMaxSlots + i, mine);
  }
  __syncthreads();  // every thread has read the epoch before thread 0 advances it
  tp_exchange_flags(peers, sync_off, rank, world, 0, &s_epoch, d_status, kSiteTpMax);
  if (i < n) {
    // NaN propagates like the packed magnitude max of the quantiser: compare the bit patterns
    // of the (non-negative) amax values as unsigned integers.
    uint32_t m = 0;
    const float* inbox = reinterpret_cast<const float*>(peers.base[rank] + box);
#pragma unroll
    for (int r = 0; r < kTpMaxWorld; ++r)
      if (r < world) m = max(m, __float_as_uint(ld_relaxed_sys_f32(inbox + r * kTpMaxSlots + i)));
    out[i] = __uint_as_float(m);
  }
}

// arg-max over a vocabulary split across ranks (the column-parallel lm_head of
// xax/arch/llm.py:970-972): every rank pushes its slice's (max, local index) per row into every
// rank's inbox, flags, and every rank picks the winner -- jnp.argmax semantics over the whole
// vocabulary: NaN counts as the maximum, the lower global index wins ties.  One CTA, rows <= 1024.
// inbox: uint2 [2][kTpMaxWorld][kTpMaxSlots], alternating by epoch parity.
__global__ void __launch_bounds__(1024) tp_argmax_kernel(const PeerTable peers, int64_t inbox_off, int64_t sync_off,
                                                         int rank, int world, int rows, int slice,
                                                         const float* __restrict__ part_max,
                                                         const int32_t* __restrict__ part_idx, int32_t* __restrict__ out,
                                                         int* d_status) {
  pdl_trigger();
  pdl_wait();
  __shared__ uint32_t s_epoch;
  const int i = threadIdx.x;
  const uint32_t* my_epoch =
      reinterpret_cast<const uint32_t*>(peers.base[rank] + sync_off) + kTpMaxSlots * kTpMaxWorld;
  const uint32_t parity = (*my_epoch + 1) & 1;
  const int64_t box = inbox_off + (int64_t)parity * kTpMaxWorld * kTpMaxSlots * 8;
  if (i < rows) {
    const unsigned long long mine =
        ((unsigned long long)(uint32_t)part_idx[i] << 32) | (unsigned long long)__float_as_uint(part_max[i]);
#pragma unroll
    for (int r = 0; r < kTpMaxWorld; ++r)
      if (r < world) {
        unsigned long long* dst = reinterpret_cast<unsigned long long*>(peers.base[r] + box) + rank * kTpMaxSlots + i;
        asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(dst), "l"(mine) : "memory");
      }
  }
  __syncthreads();  // every thread has read the epoch before thread 0 advances it
  tp_exchange_flags(peers, sync_off, rank, world, 0, &s_epoch, d_status, kSiteTpMax);
  if (i < rows) {
    const unsigned long long* inbox = reinterpret_cast<const unsigned long long*>(peers.base[rank] + box);
    float bv = 0.0f;
    int bi = 0;
#pragma unroll
    for (int r = 0; r < kTpMaxWorld; ++r) {
      if (r < world) {
        unsigned long long w;
        asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(w) : "l"(inbox + r * kTpMaxSlots + i) : "memory");
        const float v = __uint_as_float((uint32_t)w);
        const int gi = r * slice + (int)(uint32_t)(w >> 32);
        const bool vn = v != v, bn = bv != bv;
        const bool wins = r == 0 || (vn != bn ? vn : (vn ? gi < bi : (v > bv || (v == bv && gi < bi))));
        if (wins) bv = v, bi = gi;
      }
    }
    out[i] = bi;
  }
}

static int fill_peers(PeerTable& t, void* const* peer_bases, int rank, int world, const char* what) {
  if (!peer_bases || world < 1 || world > kTpMaxWorld || rank < 0 || rank >= world) {
    set_last_error("%s: needs 1 <= world <= %d, 0 <= rank < world and the table of peer mappings", what, kTpMaxWorld);
    return XAXB_BAD_ARGUMENT;
  }
  for (int r = 0; r < kTpMaxWorld; ++r) t.base[r] = nullptr;
  for (int r = 0; r < world; ++r) {
    if (!peer_bases[r] || (reinterpret_cast<uintptr_t>(peer_bases[r]) & 15)) {
      set_last_error("%s: mapping of rank %d is null or not 16-byte aligned", what, r);
      return XAXB_BAD_ARGUMENT;
    }
    t.base[r] = static_cast<uint8_t*>(peer_bases[r]);
  }
  return XAXB_OK;
}

}  // namespace xaxb

using namespace xaxb;

extern "C" {

int64_t xaxb_tp_sync_bytes(void) { return kTpSyncBytes; }

int64_t xaxb_tp_max_inbox_bytes(void) { return kTpRowMaxInboxBytes; }

int xaxb_tp_allreduce_sum_bf16(xaxb_ctx* ctx_, void* stream, void* const* peer_bases, int rank, int world,
                               int64_t data_offset_bytes, int64_t sync_offset_bytes, int64_t rows, int64_t cols,
                               void* out_bf16) {
  PeerTable t;
  int rc = fill_peers(t, peer_bases, rank, world, "tp_allreduce_sum");
  if (rc) return rc;
  if (!ctx_ || !out_bf16 || rows <= 0 || cols <= 0 || (data_offset_bytes & 15) || (sync_offset_bytes & 15) ||
      (reinterpret_cast<uintptr_t>(out_bf16) & 15)) {
    set_last_error("tp_allreduce_sum: null pointer, non-positive shape or misaligned offset");
    return XAXB_BAD_ARGUMENT;
  }
  if (rows > kTpMaxSlots || cols % 8 != 0) {
    set_last_error("tp_allreduce_sum: at most %d rows and a multiple of 8 columns", kTpMaxSlots);
    return XAXB_UNSUPPORTED;
  }
  const Ctx* ctx = reinterpret_cast<const Ctx*>(ctx_);
  launch_kernel(tp_allreduce_sum_kernel, dim3((unsigned)rows), dim3(256), 0, static_cast<cudaStream_t>(stream), 1, 
      t, data_offset_bytes, sync_offset_bytes, rank, world, (int)cols, static_cast<uint4*>(out_bf16), ctx->d_status);
  return check_launch("tp_allreduce_sum_kernel");
}

int xaxb_tp_allreduce_sum_rmsnorm(xaxb_ctx* ctx_, void* stream, void* const* peer_bases, int rank, int world,
                                  int64_t data_offset_bytes, int64_t sync_offset_bytes, int64_t rows, int64_t cols,
                                  void* x_bf16, const void* weight_bf16, float eps, void* q_e4m3, float* row_scale,
                                  float* row_inv_scale) {
  PeerTable t;
  int rc = fill_peers(t, peer_bases, rank, world, "tp_allreduce_sum_rmsnorm");
  if (rc) return rc;
  if (!ctx_ || !x_bf16 || !weight_bf16 || !q_e4m3 || !row_scale || !row_inv_scale || rows <= 0 || cols <= 0 ||
      (data_offset_bytes & 15) || (sync_offset_bytes & 15) || (reinterpret_cast<uintptr_t>(x_bf16) & 15) ||
      (reinterpret_cast<uintptr_t>(weight_bf16) & 15) || (reinterpret_cast<uintptr_t>(q_e4m3) & 7)) {
    set_last_error("tp_allreduce_sum_rmsnorm: null pointer, non-positive shape or misaligned pointer / offset");
    return XAXB_BAD_ARGUMENT;
  }
  if (rows > kTpMaxSlots || cols % 8 != 0 || cols > 256 * 4 * 8) {
    set_last_error("tp_allreduce_sum_rmsnorm: at most %d rows; columns a multiple of 8, at most 8192", kTpMaxSlots);
    return XAXB_UNSUPPORTED;
  }
  const Ctx* ctx = reinterpret_cast<const Ctx*>(ctx_);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int vec = (int)(cols / 8);
  const int vpt = (vec + 255) / 256;
  uint4* xo = static_cast<uint4*>(x_bf16);
  const uint4* wp = static_cast<const uint4*>(weight_bf16);
  uint2* qp = static_cast<uint2*>(q_e4m3);
  // the same thread layout as xaxb_rmsnorm picks for this shape, so that the sum of squares is added
  // in the same order and the bytes equal the unfused path's
#define XAXB_SUMNORM(V, N)                                                                                          \
  launch_kernel(tp_allreduce_sum_norm_kernel<V, N>, dim3((unsigned)rows), dim3(N), 0, s, 1, t, data_offset_bytes, \
                sync_offset_bytes, rank, world, vec, xo, wp, eps, qp, row_scale, row_inv_scale, ctx->d_status)
  const bool few_rows = rows <= 2 * ctx->num_sms;
  if (few_rows && vec > 256 && vec <= 512) XAXB_SUMNORM(1, 512);
  else if (few_rows && vec > 512) XAXB_SUMNORM(1, 1024);
  else if (vpt == 1) XAXB_SUMNORM(1, 256);
  else if (vpt == 2) XAXB_SUMNORM(2, 256);
  else XAXB_SUMNORM(4, 256);
#undef XAXB_SUMNORM
  return check_launch("tp_allreduce_sum_norm_kernel");
}

int64_t xaxb_tp_push_totals_bytes(void) { return (int64_t)kTpMaxSlots * 4; }

int xaxb_tp_push_sum_rmsnorm(xaxb_ctx* ctx_, void* stream, const void* staging, int64_t slot_stride_bytes,
                             const void* counter, void* totals, int world, int64_t rows, int64_t cols, void* x_bf16,
                             const void* weight_bf16, float eps, void* q_e4m3, float* row_scale,
                             float* row_inv_scale) {
  if (!ctx_ || !staging || !counter || !totals || !x_bf16 || rows <= 0 || cols <= 0 || world < 1 ||
      world > kTpMaxWorld || (slot_stride_bytes & 15) || slot_stride_bytes < rows * cols * 2 ||
      (reinterpret_cast<uintptr_t>(staging) & 15) || (reinterpret_cast<uintptr_t>(x_bf16) & 15) ||
      (reinterpret_cast<uintptr_t>(counter) & 3) || (reinterpret_cast<uintptr_t>(totals) & 3)) {
    set_last_error("tp_push_sum_rmsnorm: null pointer, bad shape, world outside 1..%d or misaligned pointer", kTpMaxWorld);
    return XAXB_BAD_ARGUMENT;
  }
  if (weight_bf16 && (!q_e4m3 || !row_scale || !row_inv_scale || (reinterpret_cast<uintptr_t>(weight_bf16) & 15) ||
                      (reinterpret_cast<uintptr_t>(q_e4m3) & 7))) {
    set_last_error("tp_push_sum_rmsnorm: with a norm weight the cast outputs are required and must be aligned");
    return XAXB_BAD_ARGUMENT;
  }
  if (rows > kTpMaxSlots || cols % 8 != 0 || cols > 256 * 4 * 8) {
    set_last_error("tp_push_sum_rmsnorm: at most %d rows; columns a multiple of 8, at most 8192", kTpMaxSlots);
    return XAXB_UNSUPPORTED;
  }
  const Ctx* ctx = reinterpret_cast<const Ctx*>(ctx_);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int vec = (int)(cols / 8);
  const int vpt = (vec + 255) / 256;
  const unsigned int pieces = (unsigned int)((long long)world * rows * vec);
  const uint8_t* st = static_cast<const uint8_t*>(staging);
  const unsigned int* cnt = static_cast<const unsigned int*>(counter);
  unsigned int* tot = static_cast<unsigned int*>(totals);
  uint4* xo = static_cast<uint4*>(x_bf16);
  const uint4* wp = static_cast<const uint4*>(weight_bf16);
  uint2* qp = static_cast<uint2*>(q_e4m3);
#define XAXB_PUSHNORM(V, N)                                                                                      \
  launch_kernel(tp_push_sum_norm_kernel<V, N>, dim3((unsigned)rows), dim3(N), 0, s, 1, st, slot_stride_bytes, cnt, \
                tot, pieces, world, vec, xo, wp, eps, qp, row_scale, row_inv_scale, ctx->d_status)
  const bool few_rows = rows <= 2 * ctx->num_sms;  // the thread layout xaxb_rmsnorm picks for this shape
  if (few_rows && vec > 256 && vec <= 512) XAXB_PUSHNORM(1, 512);
  else if (few_rows && vec > 512) XAXB_PUSHNORM(1, 1024);
  else if (vpt == 1) XAXB_PUSHNORM(1, 256);
  else if (vpt == 2) XAXB_PUSHNORM(2, 256);
  else XAXB_PUSHNORM(4, 256);
#undef XAXB_PUSHNORM
  return check_launch("tp_push_sum_norm_kernel");
}

int64_t xaxb_tp_argmax_inbox_bytes(void) { return 2ll * kTpMaxWorld * kTpMaxSlots * 8; }

int xaxb_tp_argmax(xaxb_ctx* ctx_, void* stream, void* const* peer_bases, int rank, int world,
                   int64_t inbox_offset_bytes, int64_t sync_offset_bytes, const float* part_max,
                   const int32_t* part_idx, int64_t rows, int64_t slice, int32_t* out) {
  PeerTable t;
  int rc = fill_peers(t, peer_bases, rank, world, "tp_argmax");
  if (rc) return rc;
  if (!ctx_ || !part_max || !part_idx || !out || rows <= 0 || slice <= 0 || (inbox_offset_bytes & 15) ||
      (sync_offset_bytes & 15)) {
    set_last_error("tp_argmax: null pointer, non-positive size or misaligned offset");
    return XAXB_BAD_ARGUMENT;
  }
  if (rows > kTpMaxSlots || slice * (int64_t)world > 2147483647ll) {
    set_last_error("tp_argmax: at most %d rows and a vocabulary below 2^31", kTpMaxSlots);
    return XAXB_UNSUPPORTED;
  }
  const Ctx* ctx = reinterpret_cast<const Ctx*>(ctx_);
  const unsigned threads = (unsigned)((rows + 31) / 32 * 32);
  launch_kernel(tp_argmax_kernel, dim3(1), dim3(threads), 0, static_cast<cudaStream_t>(stream), 1, 
      t, inbox_offset_bytes, sync_offset_bytes, rank, world, (int)rows, (int)slice, part_max, part_idx, out,
      ctx->d_status);
  return check_launch("tp_argmax_kernel");
}

int xaxb_tp_allreduce_max_f32(xaxb_ctx* ctx_, void* stream, void* const* peer_bases, int rank, int world,
                              int64_t inbox_offset_bytes, int64_t sync_offset_bytes, const float* in, float* out,
                              int64_t n) {
  PeerTable t;
  int rc = fill_peers(t, peer_bases, rank, world, "tp_allreduce_max");
  if (rc) return rc;
  if (!ctx_ || !in || !out || n <= 0 || (inbox_offset_bytes & 15) || (sync_offset_bytes & 15)) {
    set_last_error("tp_allreduce_max: null pointer, non-positive size or misaligned offset");
    return XAXB_BAD_ARGUMENT;
  }
  if (n > kTpMaxSlots) {
    set_last_error("tp_allreduce_max: at most %d values", kTpMaxSlots);
    return XAXB_UNSUPPORTED;
  }
  const Ctx* ctx = reinterpret_cast<const Ctx*>(ctx_);
  const unsigned threads = (unsigned)((n + 31) / 32 * 32) < 32u ? 32u : (unsigned)((n + 31) / 32 * 32);
  launch_kernel(tp_allreduce_max_kernel, dim3(1), dim3(threads), 0, static_cast<cudaStream_t>(stream), 1, 
      t, inbox_offset_bytes, sync_offset_bytes, rank, world, (int)n, in, out, ctx->d_status);
  return check_launch("tp_allreduce_max_kernel");
}

}  // extern "C"
