// Kernel 2: e4m3 x e4m3 (and bf16 x bf16) GEMM on the 5th-generation tensor cores.
//
//   out[m, n] = bf16( acc[m, n] * row_mul[m] * col_mul[n] + bias[n] + residual[m, n] )
//   acc[m, n] = sum_k a[m, k] * b[n, k]           (float32 accumulators in tensor memory)
//
// Both operands are K-contiguous (activations [M, K], weights [N, K]), which is the K-major
// layout tcgen05.mma reads straight from shared memory.  One persistent CTA per SM:
//   warp 0    TMA producer: 128-byte-swizzled tiles of A (128 x 128 B) and B (BN x 128 B)
//             into a ring of shared-memory stages, completion on "full" mbarriers;
//   warp 1    MMA issuer: one thread issues 4 tcgen05.mma (K = 32 bytes each) per stage into
//             one of two TMEM accumulators; tcgen05.commit releases the stage ("empty") and,
//             after the last K block, publishes the accumulator ("acc_full");
//   warps 2-5 epilogue: tcgen05.ld the finished accumulator (thread = row), apply the
//             dequantisation multipliers, bias and residual, cast to bf16 and store; then
//             hand the accumulator back ("acc_empty") so the next tile's main loop overlaps.
// Tiles whose rows or columns run past M / N / K rely on TMA's zero fill; stores are guarded.
#include "common.cuh"

namespace xaxb {

constexpr int kBM = 128;          // rows of A per tile = UMMA M
constexpr int kBKBytes = 128;     // K bytes per stage = one swizzle span
constexpr int kGemmThreads = 192; // 6 warps
constexpr int kSiteProducer = 1, kSiteMma = 2, kSiteEpilogue = 3, kSiteMmaAcc = 4;

struct GemmParams {
  int M, N, K;
  int num_k_blocks;
  int tiles_m, tiles_n;
  const float* row_mul;
  int row_mul_stride;
  const float* col_mul;
  int col_mul_stride;
  const __nv_bfloat16* bias;
  const __nv_bfloat16* residual;
  long long ldr;
  __nv_bfloat16* out;
  long long ldo;
  int* d_status;
};

template <int BN>
struct GemmCfg {
  static constexpr int kStageBytes = kBM * kBKBytes + BN * kBKBytes;
  static constexpr int kStages = (200 * 1024) / kStageBytes > 12 ? 12 : (200 * 1024) / kStageBytes;
  static constexpr int kTmemCols = 2 * BN < 32 ? 32 : 2 * BN;
  static constexpr int kSmemBytes = kStages * kStageBytes + 1024 /*alignment slack*/ + 256 /*barriers*/;
};

template <int BN, bool IS_FP8>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
               const GemmParams p) {
  using Cfg = GemmCfg<BN>;
  constexpr int kStages = Cfg::kStages;
  constexpr int kElemBytes = IS_FP8 ? 1 : 2;
  constexpr int kBKElems = kBKBytes / kElemBytes;
  constexpr uint32_t kIdesc = umma_idesc(IS_FP8 ? kFmtE4M3 : kFmtBF16, IS_FP8 ? kFmtE4M3 : kFmtBF16, 0, 0, kBM, BN);

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* smem_a = smem;                                  // kStages x 16 KiB
  uint8_t* smem_b = smem + kStages * kBM * kBKBytes;       // kStages x BN*128 B
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kStages * Cfg::kStageBytes);
  uint64_t* full = bars;                 // [kStages]
  uint64_t* empty = bars + kStages;      // [kStages]
  uint64_t* acc_full = bars + 2 * kStages;   // [2]
  uint64_t* acc_empty = acc_full + 2;        // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(full + s, 1);
      mbar_init(empty + s, 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(acc_full + i, 1);
      mbar_init(acc_empty + i, 4);  // one arrival per epilogue warp
    }
    *abort_flag = 0;
    fence_mbar_init();
    prefetch_tmap(&tmap_a);
    prefetch_tmap(&tmap_b);
  }
  if (warp == 2) {
    tmem_alloc(tmem_slot, Cfg::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  const int num_tiles = p.tiles_m * p.tiles_n;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        const int m0 = (tile % p.tiles_m) * kBM;
        const int n0 = (tile / p.tiles_m) * BN;
        for (int kb = 0; kb < p.num_k_blocks; ++kb) {
          ok = mbar_wait(empty + stage, phase ^ 1, abort_flag, p.d_status, XAXB_DEVICE_TIMEOUT * 1000 + kSiteProducer);
          if (!ok) break;
          mbar_arrive_expect_tx(full + stage, Cfg::kStageBytes);
          tma_load_2d(smem_a + stage * kBM * kBKBytes, &tmap_a, full + stage, kb * kBKElems, m0);
          tma_load_2d(smem_b + stage * BN * kBKBytes, &tmap_b, full + stage, kb * kBKElems, n0);
          if (++stage == kStages) stage = 0, phase ^= 1;
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        ok = mbar_wait(acc_empty + acc, acc_phase ^ 1, abort_flag, p.d_status,
                       XAXB_DEVICE_TIMEOUT * 1000 + kSiteMmaAcc);
        if (!ok) break;
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < p.num_k_blocks; ++kb) {
          ok = mbar_wait(full + stage, phase, abort_flag, p.d_status, XAXB_DEVICE_TIMEOUT * 1000 + kSiteMma);
          if (!ok) break;
          tc_fence_after_sync();
          const uint64_t a_desc = umma_desc_kmajor_sw128(smem_u32(smem_a + stage * kBM * kBKBytes));
          const uint64_t b_desc = umma_desc_kmajor_sw128(smem_u32(smem_b + stage * BN * kBKBytes));
#pragma unroll
          for (int k = 0; k < kBKBytes / 32; ++k) {
            // advancing the start address by 32 bytes (>> 4 = 2) walks K inside the swizzle span
            if (IS_FP8)
              umma_f8(d_tmem, a_desc + 2 * k, b_desc + 2 * k, kIdesc, (kb | k) != 0);
            else
              umma_f16(d_tmem, a_desc + 2 * k, b_desc + 2 * k, kIdesc, (kb | k) != 0);
          }
          umma_commit(empty + stage);  // frees the stage once these MMAs have read it
          if (++stage == kStages) stage = 0, phase ^= 1;
        }
        if (!ok) break;
        umma_commit(acc_full + acc);  // accumulator complete
        if (++acc == 2) acc = 0, acc_phase ^= 1;
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..5)
    const int quarter = warp & 3;          // TMEM lanes this warp may read
    const int row_in_tile = quarter * 32 + lane;
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
      const int m0 = (tile % p.tiles_m) * kBM;
      const int n0 = (tile / p.tiles_m) * BN;
      ok = mbar_wait(acc_full + acc, acc_phase, abort_flag, p.d_status, XAXB_DEVICE_TIMEOUT * 1000 + kSiteEpilogue);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after_sync();
      const int m = m0 + row_in_tile;
      const bool row_ok = m < p.M;
      const float rm = (row_ok && p.row_mul) ? p.row_mul[(long long)m * p.row_mul_stride] : 1.0f;
      const uint32_t taddr = tmem_base + (uint32_t(quarter * 32) << 16) + acc * BN;
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += 32) {
        uint32_t r[32];
        tmem_ld_x32(taddr + c0, r);
        tmem_ld_wait();
        const int nbase = n0 + c0;
        if (row_ok && nbase < p.N) {
          __nv_bfloat16* orow = p.out + (long long)m * p.ldo + nbase;
          const __nv_bfloat16* rrow = p.residual ? p.residual + (long long)m * p.ldr + nbase : nullptr;
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            const int n = nbase + v * 8;
            if (n >= p.N) break;  // N is a multiple of 8: whole vectors only
            float f[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              float x = __uint_as_float(r[v * 8 + j]) * rm;
              if (p.col_mul) x *= __ldg(p.col_mul + (long long)(n + j) * p.col_mul_stride);
              f[j] = x;
            }
            if (p.bias) {
              const uint4 bv = __ldg(reinterpret_cast<const uint4*>(p.bias + n));
              const uint32_t bw[4] = {bv.x, bv.y, bv.z, bv.w};
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                f[2 * j] += bf16_bits_to_float(bw[j] & 0xFFFFu);
                f[2 * j + 1] += bf16_bits_to_float(bw[j] >> 16);
              }
            }
            if (rrow) {
              const uint4 rv = *reinterpret_cast<const uint4*>(rrow + v * 8);
              const uint32_t rw[4] = {rv.x, rv.y, rv.z, rv.w};
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                f[2 * j] += bf16_bits_to_float(rw[j] & 0xFFFFu);
                f[2 * j + 1] += bf16_bits_to_float(rw[j] >> 16);
              }
            }
            uint4 o;
            uint32_t* ow = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const uint32_t lo = __bfloat16_as_ushort(__float2bfloat16_rn(f[2 * j]));
              const uint32_t hi = __bfloat16_as_ushort(__float2bfloat16_rn(f[2 * j + 1]));
              ow[j] = lo | (hi << 16);
            }
            *reinterpret_cast<uint4*>(orow + v * 8) = o;
          }
        }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(acc_empty + acc);
      if (++acc == 2) acc = 0, acc_phase ^= 1;
    }
  }

  // ---------------------------------------------------------------------- teardown
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 2) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, Cfg::kTmemCols);
  }
}

template <int BN, bool IS_FP8>
static int launch_gemm(const Ctx* ctx, cudaStream_t stream, const void* a, long long lda_bytes, const void* b,
                       long long ldb_bytes, GemmParams& p) {
  using Cfg = GemmCfg<BN>;
  constexpr int kElemBytes = IS_FP8 ? 1 : 2;
  CUtensorMap ta, tb;
  int rc = make_tmap_2d(ctx, &ta, a, kElemBytes, (uint64_t)p.K, (uint64_t)p.M, (uint64_t)lda_bytes,
                        kBKBytes / kElemBytes, kBM);
  if (rc) return rc;
  rc = make_tmap_2d(ctx, &tb, b, kElemBytes, (uint64_t)p.K, (uint64_t)p.N, (uint64_t)ldb_bytes, kBKBytes / kElemBytes,
                    BN);
  if (rc) return rc;
  p.tiles_m = (p.M + kBM - 1) / kBM;
  p.tiles_n = (p.N + BN - 1) / BN;
  p.num_k_blocks = (int)(((long long)p.K * kElemBytes + kBKBytes - 1) / kBKBytes);
  static bool attr_set = false;  // per template instantiation
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(gemm_tc_kernel<BN, IS_FP8>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         Cfg::kSmemBytes);
    if (e != cudaSuccess) {
      set_last_error("gemm: cudaFuncSetAttribute(%d bytes): %s", Cfg::kSmemBytes, cudaGetErrorString(e));
      return XAXB_LAUNCH_FAILED;
    }
    attr_set = true;
  }
  const int tiles = p.tiles_m * p.tiles_n;
  const int grid = tiles < ctx->num_sms ? tiles : ctx->num_sms;
  gemm_tc_kernel<BN, IS_FP8><<<grid, kGemmThreads, Cfg::kSmemBytes, stream>>>(ta, tb, p);
  return check_launch("gemm_tc_kernel");
}

// Tile width: the widest N tile that still gives every SM a tile.
static int pick_bn(long long M, long long N, int num_sms) {
  const long long tiles_m = (M + kBM - 1) / kBM;
  const int cand[4] = {256, 128, 64, 32};
  for (int i = 0; i < 4; ++i) {
    const long long tiles = tiles_m * ((N + cand[i] - 1) / cand[i]);
    if (tiles >= num_sms || i == 3) return cand[i];
  }
  return 32;
}

template <bool IS_FP8>
static int gemm_entry(xaxb_ctx* ctx_, void* stream, const void* a, int64_t lda, const void* b, int64_t ldb, int64_t M,
                      int64_t N, int64_t K, const float* row_mul, int row_mul_stride, const float* col_mul,
                      int col_mul_stride, const void* bias, const void* residual, int64_t ldr, void* out,
                      int64_t ldo) {
  if (!ctx_ || !a || !b || !out || M <= 0 || N <= 0 || K <= 0) {
    set_last_error("gemm: null pointer or non-positive shape");
    return XAXB_BAD_ARGUMENT;
  }
  constexpr int eb = IS_FP8 ? 1 : 2;
  if ((K * eb) % 16 != 0 || N % 8 != 0 || ldo % 8 != 0 || (residual && ldr % 8 != 0) ||
      (reinterpret_cast<uintptr_t>(out) & 15) || (reinterpret_cast<uintptr_t>(bias) & 15) ||
      (reinterpret_cast<uintptr_t>(residual) & 15) || M > 0x7fffffff || N > 0x7fffffff || K > 0x7fffffff) {
    set_last_error("gemm: K bytes (%lld) must be a multiple of 16; N, ldo, ldr multiples of 8; out/bias/residual "
                   "16-byte aligned", (long long)(K * eb));
    return XAXB_BAD_ARGUMENT;
  }
  const Ctx* ctx = reinterpret_cast<const Ctx*>(ctx_);
  GemmParams p;
  p.M = (int)M, p.N = (int)N, p.K = (int)K;
  p.row_mul = row_mul, p.row_mul_stride = row_mul_stride;
  p.col_mul = col_mul, p.col_mul_stride = col_mul_stride;
  p.bias = static_cast<const __nv_bfloat16*>(bias);
  p.residual = static_cast<const __nv_bfloat16*>(residual);
  p.ldr = ldr;
  p.out = static_cast<__nv_bfloat16*>(out);
  p.ldo = ldo;
  p.d_status = ctx->d_status;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  switch (pick_bn(M, N, ctx->num_sms)) {
    case 256: return launch_gemm<256, IS_FP8>(ctx, s, a, lda * eb, b, ldb * eb, p);
    case 128: return launch_gemm<128, IS_FP8>(ctx, s, a, lda * eb, b, ldb * eb, p);
    case 64: return launch_gemm<64, IS_FP8>(ctx, s, a, lda * eb, b, ldb * eb, p);
    default: return launch_gemm<32, IS_FP8>(ctx, s, a, lda * eb, b, ldb * eb, p);
  }
}

}  // namespace xaxb

using namespace xaxb;

extern "C" {

int xaxb_gemm_fp8(xaxb_ctx* ctx, void* stream, const void* a_e4m3, int64_t lda, const void* b_e4m3, int64_t ldb,
                  int64_t M, int64_t N, int64_t K, const float* row_mul, int row_mul_stride, const float* col_mul,
                  int col_mul_stride, const void* bias_bf16, const void* residual_bf16, int64_t ldr, void* out_bf16,
                  int64_t ldo) {
  return gemm_entry<true>(ctx, stream, a_e4m3, lda, b_e4m3, ldb, M, N, K, row_mul, row_mul_stride, col_mul,
                          col_mul_stride, bias_bf16, residual_bf16, ldr, out_bf16, ldo);
}

int xaxb_gemm_bf16(xaxb_ctx* ctx, void* stream, const void* a_bf16, int64_t lda, const void* b_bf16, int64_t ldb,
                   int64_t M, int64_t N, int64_t K, const float* row_mul, int row_mul_stride, const float* col_mul,
                   int col_mul_stride, const void* bias_bf16, const void* residual_bf16, int64_t ldr, void* out_bf16,
                   int64_t ldo) {
  return gemm_entry<false>(ctx, stream, a_bf16, lda, b_bf16, ldb, M, N, K, row_mul, row_mul_stride, col_mul,
                           col_mul_stride, bias_bf16, residual_bf16, ldr, out_bf16, ldo);
}

}  // extern "C"
