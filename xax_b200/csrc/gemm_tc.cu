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
#include <cstdio>
#include <cstdlib>

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
  // OR-ed into the MMA instruction descriptor: the operand formats when they are not e4m3 (bit 7 = A is e5m2,
  // bit 10 = B is e5m2; the f8f6f4 kind mixes the two freely).  0 for e4m3 x e4m3 and for bf16.
  uint32_t idesc_or;
  // The launch may overlap the previous kernel (programmatic dependent launch).  Operand B -- the
  // weights of a linear layer -- is never written by a kernel of the same stream section, so the
  // producer may fetch it before it waits for the previous kernel:
  // it asks L2 for the first `prefetch_l2` K blocks of B there (0: nothing ahead of the wait).
  // (Requests further ahead than that do not pay: an SM keeps about 42 KB in flight whatever the
  // depth of its shared-memory ring, and a request to L2 occupies that budget like a load does --
  // asking 8 to 64 blocks ahead while streaming made every decode shape 3 to 50 % slower.)
  int prefetch_l2;
  int band;        // tile rows per band of the tile order (see tile_coords)
  // Tensor-parallel push (split-K kernel only): with push_world > 0 the epilogue writes every 16-byte
  // piece of the output to push_out[r] for each rank r < push_world (this rank's slot of rank r's
  // staging buffer; plain peer stores over NVLink) instead of `out`, and when a CTA's pieces are all
  // written it adds their number to push_flag[r] on every rank with a system-scope release.
  __nv_bfloat16* push_out[8];
  unsigned int* push_flag[8];
  int push_world;
  // Cross-entropy epilogue (gemm_tc_kernel, tiles of 64 columns and more): with ce_part set the output
  // tile is never stored.  Each epilogue thread owns a row and reduces the tile's columns of that row --
  // the logits of a vocabulary slice -- to (max, sum of exp(logit - max), the logit of column
  // ce_targets[row] if it lies in the tile else -inf, the column of the max) and writes that to
  // ce_part[row * tiles_n + tile column]; a second kernel merges the slices of a row.
  float4* ce_part;
  const int32_t* ce_targets;
};

// Tile order: bands of kBand tile rows, column by column inside a band (row index fastest).  The
// tiles in flight at any moment then share a few row blocks of A and a few column blocks of B
// -- a working set that stays in L2 -- instead of sweeping all of A for every column of tiles.
__device__ __forceinline__ void tile_coords(int kBand, int tile, int tiles_m, int tiles_n, int& tm, int& tn) {
  const int per_band = kBand * tiles_n;
  const int band = tile / per_band, r = tile - band * per_band;
  const int rows = min(kBand, tiles_m - band * kBand);
  tn = r / rows;
  tm = band * kBand + (r - tn * rows);
}

// Default number of K blocks of operand B that a producer asks L2 for ahead of the wait on the
// previous kernel (GemmParams::prefetch_l2).
constexpr int kMaxPrefetchBlocks = 4;

template <int BN>
struct GemmCfg {
  static constexpr int kStageBytes = kBM * kBKBytes + BN * kBKBytes;
  // epilogue staging.  BN >= 64: a [128 x 64] bf16 block in TMA-store layout (128-byte rows,
  // swizzled) plus per-tile column multipliers and bias; BN = 32: a [128 x 32] float32 slab with
  // padded rows for the coalesced direct-store path.
  static constexpr bool kTmaStore = BN >= 64;
  static constexpr int kEpiCols = 32;
  static constexpr int kEpiRowFloats = kEpiCols + 4;
  static constexpr int kEpiBytes = kTmaStore ? (kBM * 128 + 2 * BN * 4) : (kBM * kEpiRowFloats * 4);
  static constexpr int kStagesFit = (224 * 1024 - kEpiBytes) / kStageBytes;
  static constexpr int kStages = kStagesFit > 12 ? 12 : kStagesFit;
  static constexpr int kTmemCols = 2 * BN < 32 ? 32 : 2 * BN;
  static constexpr int kSmemBytes = kStages * kStageBytes + kEpiBytes + 1024 /*alignment slack*/ + 256 /*barriers*/;
};

// f[j] *= row multiplier * column multiplier of column n + j (n a multiple of 8)
__device__ __forceinline__ void apply_muls(float (&f)[8], float rm, const float* col_mul, int col_mul_stride, int n) {
  if (!col_mul) {
#pragma unroll
    for (int j = 0; j < 8; ++j) f[j] *= rm;
  } else if (col_mul_stride == 0) {
    const float c = __ldg(col_mul) * rm;
#pragma unroll
    for (int j = 0; j < 8; ++j) f[j] *= c;
  } else if (col_mul_stride == 1 && (reinterpret_cast<uintptr_t>(col_mul) & 15) == 0) {
    const float4 a = __ldg(reinterpret_cast<const float4*>(col_mul + n));
    const float4 b = __ldg(reinterpret_cast<const float4*>(col_mul + n + 4));
    f[0] *= rm * a.x, f[1] *= rm * a.y, f[2] *= rm * a.z, f[3] *= rm * a.w;
    f[4] *= rm * b.x, f[5] *= rm * b.y, f[6] *= rm * b.z, f[7] *= rm * b.w;
  } else {
#pragma unroll
    for (int j = 0; j < 8; ++j) f[j] *= rm * __ldg(col_mul + (long long)(n + j) * col_mul_stride);
  }
}

// all-of vote over the 128 epilogue threads on named barrier 1
__device__ __forceinline__ bool epilogue_all(bool pred) {
  uint32_t r;
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t"
      "setp.ne.u32 q, %1, 0;\n\t"
      "bar.red.and.pred p, 1, 128, q;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(r)
      : "r"((uint32_t)pred)
      : "memory");
  return r != 0;
}

__device__ __forceinline__ void epilogue_sync() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

template <int BN, bool IS_FP8>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
               const __grid_constant__ CUtensorMap tmap_out, const GemmParams p) {
  using Cfg = GemmCfg<BN>;
  constexpr int kStages = Cfg::kStages;
  constexpr int kElemBytes = IS_FP8 ? 1 : 2;
  constexpr int kBKElems = kBKBytes / kElemBytes;
  constexpr uint32_t kIdesc = umma_idesc(IS_FP8 ? kFmtE4M3 : kFmtBF16, IS_FP8 ? kFmtE4M3 : kFmtBF16, 0, 0, kBM, BN);

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* smem_a = smem;                                  // kStages x 16 KiB
  uint8_t* smem_b = smem + kStages * kBM * kBKBytes;       // kStages x BN*128 B
  float* estage = reinterpret_cast<float*>(smem + kStages * Cfg::kStageBytes);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kStages * Cfg::kStageBytes + Cfg::kEpiBytes);
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
  pdl_trigger();  // tensor memory is allocated: the next kernel may be scheduled

  const int num_tiles = p.tiles_m * p.tiles_n;
  // Everything that reads or writes global memory waits for the previous kernel in the stream;
  // the producer thread first asks L2 for operand B of its first tile (below).
  if (threadIdx.x != 0) pdl_wait();

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      // While the previous kernel is still running, bring in operand B of this CTA's first tile
      // (the weights: what a decode-sized GEMM streams from HBM).  L2 is the point of coherence and
      // nothing in flight writes B, so this is safe whatever precedes the kernel.
      if (p.prefetch_l2 && (int)blockIdx.x < num_tiles) {
        int tm, tn;
        tile_coords(p.band, (int)blockIdx.x, p.tiles_m, p.tiles_n, tm, tn);
        int kk = (int)(((long long)blockIdx.x * 5) % p.num_k_blocks);
        const int n_l2 = min(p.num_k_blocks, p.prefetch_l2);
        for (int i = 0; i < n_l2; ++i) {
          tma_prefetch_l2_2d(&tmap_b, kk * kBKElems, tn * BN);
          if (++kk == p.num_k_blocks) kk = 0;
        }
      }
      pdl_wait();
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        int tm, tn;
        tile_coords(p.band, tile, p.tiles_m, p.tiles_n, tm, tn);
        const int m0 = tm * kBM, n0 = tn * BN;
        // Each tile walks K from its own starting block: CTAs that share an operand tile (all
        // N tiles read the same rows of A) then ask L2 for different lines at any moment.
        int kk = (int)(((long long)tile * 5) % p.num_k_blocks);
        for (int kb = 0; kb < p.num_k_blocks; ++kb) {
          ok = mbar_wait(empty + stage, phase ^ 1, abort_flag, p.d_status, XAXB_DEVICE_TIMEOUT * 1000 + kSiteProducer);
          if (!ok) break;
          mbar_arrive_expect_tx(full + stage, Cfg::kStageBytes);
          tma_load_2d(smem_a + stage * kBM * kBKBytes, &tmap_a, full + stage, kk * kBKElems, m0);
          tma_load_2d(smem_b + stage * BN * kBKBytes, &tmap_b, full + stage, kk * kBKElems, n0);
          if (++kk == p.num_k_blocks) kk = 0;
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
              umma_f8(d_tmem, a_desc + 2 * k, b_desc + 2 * k, kIdesc | p.idesc_or, (kb | k) != 0);
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
    // Per slab of kEpiCols columns: (A) thread = row pulls its accumulator values out of TMEM
    // and parks them in shared memory; (B) work item = (row, 8 consecutive columns), consecutive
    // threads take consecutive column groups of a row, so the residual read and the bf16 store
    // are contiguous 128-byte runs instead of one 16-byte piece per row.
    if constexpr (Cfg::kTmaStore) {
      // TMA-store epilogue.  Per 64-column block: thread = row reads its accumulator values from
      // TMEM, applies row/column multipliers, bias and residual, packs to bf16 and writes its
      // 128-byte row into a swizzled staging block; one thread then hands the block to the TMA
      // unit, which writes full rows to global memory and clips rows / columns past M / N.
      uint8_t* stage_out = reinterpret_cast<uint8_t*>(estage);
      float* cmul_s = reinterpret_cast<float*>(stage_out + kBM * 128);
      float* bias_s = cmul_s + BN;
      const int quarter = warp & 3;
      const int row_in_tile = quarter * 32 + lane;
      const int t = threadIdx.x - 64;
      int acc = 0;
      uint32_t acc_phase = 0;
      if (t == 0) prefetch_tmap(&tmap_out);
      for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x) {
        int tm, tn;
        tile_coords(p.band, tile, p.tiles_m, p.tiles_n, tm, tn);
        const int m0 = tm * kBM, n0 = tn * BN;
        // The tile's multipliers and bias are fetched while its main loop is still running (every
        // thread passed the previous tile's last barrier after its last read of cmul_s / bias_s).
        for (int i = t; i < BN; i += 128) {
          const int n = n0 + i;
          float cm = 0.0f, bs = 0.0f;
          if (n < p.N) {
            cm = p.col_mul ? __ldg(p.col_mul + (long long)n * p.col_mul_stride) : 1.0f;
            bs = p.bias ? __bfloat162float(p.bias[n]) : 0.0f;
          }
          cmul_s[i] = cm;
          bias_s[i] = bs;
        }
        const int m = m0 + row_in_tile;
        const bool row_ok = m < p.M;
        const float rm = (row_ok && p.row_mul) ? __ldg(p.row_mul + (long long)m * p.row_mul_stride) : 1.0f;
        bool ok = mbar_wait(acc_full + acc, acc_phase, abort_flag, p.d_status, XAXB_DEVICE_TIMEOUT * 1000 + kSiteEpilogue);
        if (!epilogue_all(ok)) break;  // (also publishes cmul_s / bias_s)
        tc_fence_after_sync();
        const uint32_t taddr = tmem_base + (uint32_t(quarter * 32) << 16) + acc * BN;
        if (p.ce_part) {
          const int tgt = row_ok ? p.ce_targets[m] : -1;
          float mx = -INFINITY, l = 0.0f, tv = -INFINITY;
          int best = 0x7fffffff;
#pragma unroll 1
          for (int c0 = 0; c0 < BN; c0 += 32) {
            uint32_t r[32];
            tmem_ld_x32(taddr + c0, r);
            tmem_ld_wait();
            if (c0 + 32 >= BN) {  // accumulator fully read: hand it back to the MMA warp
              tc_fence_before_sync();
              __syncwarp();
              if (lane == 0) mbar_arrive(acc_empty + acc);
            }
            float f[32];
            float cmx = -INFINITY;
            int cidx = 0x7fffffff;
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              const int n = n0 + c0 + i;
              f[i] = n < p.N ? fmaf(__uint_as_float(r[i]) * rm, cmul_s[c0 + i], bias_s[c0 + i]) : -INFINITY;
              if (f[i] > cmx) cmx = f[i], cidx = n;  // strictly greater: the first index wins a tie
              if (n == tgt) tv = f[i];
            }
            if (cmx > mx) {
              l *= expf(mx - cmx);  // (mx = -inf on the first chunk: l is 0 and stays 0)
              mx = cmx;
              best = cidx;
            }
#pragma unroll
            for (int i = 0; i < 32; ++i) l += expf(f[i] - mx);
          }
          if (row_ok) p.ce_part[(long long)m * p.tiles_n + tn] = make_float4(mx, l, tv, __int_as_float(best));
          epilogue_sync();  // every thread has read cmul_s / bias_s before the next tile overwrites them
          if (++acc == 2) acc = 0, acc_phase ^= 1;
          continue;
        }
#pragma unroll 1
        for (int c0 = 0; c0 < BN; c0 += 64) {
          // the TMA unit must have finished reading the staging block of the previous store
          if (t == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
          epilogue_sync();  // (also publishes cmul_s / bias_s on the first block)
#pragma unroll
          for (int h = 0; h < 64; h += 32) {
            uint32_t r[32];
            tmem_ld_x32(taddr + c0 + h, r);
            tmem_ld_wait();
            if (c0 + 64 >= BN && h == 32) {  // accumulator fully read: hand it back to the MMA warp
              tc_fence_before_sync();
              __syncwarp();
              if (lane == 0) mbar_arrive(acc_empty + acc);
            }
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              const int cc = c0 + h + v * 8;  // column within the tile
              float f[8];
              {  // column multipliers and bias of the eight columns: four 16-byte shared-memory reads
                const float4 ca = *reinterpret_cast<const float4*>(cmul_s + cc), cb = *reinterpret_cast<const float4*>(cmul_s + cc + 4);
                const float4 ba = *reinterpret_cast<const float4*>(bias_s + cc), bb = *reinterpret_cast<const float4*>(bias_s + cc + 4);
                const float cm[8] = {ca.x, ca.y, ca.z, ca.w, cb.x, cb.y, cb.z, cb.w};
                const float bs[8] = {ba.x, ba.y, ba.z, ba.w, bb.x, bb.y, bb.z, bb.w};
#pragma unroll
                for (int j = 0; j < 8; ++j) f[j] = fmaf(__uint_as_float(r[v * 8 + j]) * rm, cm[j], bs[j]);
              }
              if (p.residual && row_ok && n0 + cc < p.N) {
                const uint4 rv = *reinterpret_cast<const uint4*>(p.residual + (long long)m * p.ldr + n0 + cc);
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
                const uint32_t lo16 = __bfloat16_as_ushort(__float2bfloat16_rn(f[2 * j]));
                const uint32_t hi16 = __bfloat16_as_ushort(__float2bfloat16_rn(f[2 * j + 1]));
                ow[j] = lo16 | (hi16 << 16);
              }
              *reinterpret_cast<uint4*>(stage_out + sw128_offset(row_in_tile, (h + v * 8) / 8)) = o;
            }
          }
          fence_proxy_async_smem();
          epilogue_sync();
          if (t == 0 && n0 + c0 < p.N) {
            asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
                         ::"l"(&tmap_out), "r"(smem_u32(stage_out)), "r"(n0 + c0), "r"(m0)
                         : "memory");
            asm volatile("cp.async.bulk.commit_group;" ::: "memory");
          }
        }
        if (++acc == 2) acc = 0, acc_phase ^= 1;
      }
      if (t == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");  // stores done before the CTA leaves
    } else {
    constexpr int kEpiCols = Cfg::kEpiCols, kRowF = Cfg::kEpiRowFloats, kGroups = kEpiCols / 8;
    const int quarter = warp & 3;          // TMEM lanes this warp may read
    const int row_in_tile = quarter * 32 + lane;
    const int t = threadIdx.x - 64;        // 0..127
    int acc = 0;
    uint32_t acc_phase = 0;
    for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x) {
      int tm, tn;
      tile_coords(p.band, tile, p.tiles_m, p.tiles_n, tm, tn);
      const int m0 = tm * kBM, n0 = tn * BN;
      bool ok = mbar_wait(acc_full + acc, acc_phase, abort_flag, p.d_status, XAXB_DEVICE_TIMEOUT * 1000 + kSiteEpilogue);
      if (!epilogue_all(ok)) break;
      tc_fence_after_sync();
      const uint32_t taddr = tmem_base + (uint32_t(quarter * 32) << 16) + acc * BN;
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += kEpiCols) {
        float* srow = estage + row_in_tile * kRowF;
#pragma unroll
        for (int h = 0; h < kEpiCols; h += 32) {
          uint32_t r[32];
          tmem_ld_x32(taddr + c0 + h, r);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; i += 4)
            *reinterpret_cast<float4*>(srow + h + i) = make_float4(__uint_as_float(r[i]), __uint_as_float(r[i + 1]),
                                                                   __uint_as_float(r[i + 2]), __uint_as_float(r[i + 3]));
        }
        if (c0 + kEpiCols >= BN) {  // the accumulator has been read out: the MMA warp may reuse it
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive(acc_empty + acc);
        }
        epilogue_sync();
        // items of this thread in the slab: (row, 8 columns); residual pieces are fetched first
        // so their latency overlaps instead of adding up
        constexpr int kItems = kBM * kGroups / 128;
        uint4 resv[kItems];
#pragma unroll
        for (int k = 0; k < kItems; ++k) {
          const int it = t + k * 128;
          const int m = m0 + it / kGroups, n = n0 + c0 + (it % kGroups) * 8;
          resv[k] = make_uint4(0, 0, 0, 0);
          if (p.residual && m < p.M && n < p.N)
            resv[k] = *reinterpret_cast<const uint4*>(p.residual + (long long)m * p.ldr + n);
        }
#pragma unroll
        for (int k = 0; k < kItems; ++k) {
          const int it = t + k * 128;
          const int rr = it / kGroups, g8 = it % kGroups;
          const int m = m0 + rr, n = n0 + c0 + g8 * 8;
          if (m >= p.M || n >= p.N) continue;
          const float4 lo = *reinterpret_cast<const float4*>(estage + rr * kRowF + g8 * 8);
          const float4 hi = *reinterpret_cast<const float4*>(estage + rr * kRowF + g8 * 8 + 4);
          float f[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
          const float rm = p.row_mul ? __ldg(p.row_mul + (long long)m * p.row_mul_stride) : 1.0f;
          apply_muls(f, rm, p.col_mul, p.col_mul_stride, n);
          if (p.bias) {
            const uint4 bv = __ldg(reinterpret_cast<const uint4*>(p.bias + n));
            const uint32_t bw[4] = {bv.x, bv.y, bv.z, bv.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              f[2 * j] += bf16_bits_to_float(bw[j] & 0xFFFFu);
              f[2 * j + 1] += bf16_bits_to_float(bw[j] >> 16);
            }
          }
          if (p.residual) {
            const uint32_t rw[4] = {resv[k].x, resv[k].y, resv[k].z, resv[k].w};
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
            const uint32_t lo16 = __bfloat16_as_ushort(__float2bfloat16_rn(f[2 * j]));
            const uint32_t hi16 = __bfloat16_as_ushort(__float2bfloat16_rn(f[2 * j + 1]));
            ow[j] = lo16 | (hi16 << 16);
          }
          *reinterpret_cast<uint4*>(p.out + (long long)m * p.ldo + n) = o;
        }
        epilogue_sync();  // the slab is free for the next columns
      }
      if (++acc == 2) acc = 0, acc_phase ^= 1;
    }
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

// ---------------------------------------------------------------------------------------
// Split-K variant for M <= 128 (decode): weight streaming.  A thread-block cluster of S CTAs
// shares one [128 x BN] output tile; CTA r multiplies K slice r into its own TMEM accumulator,
// parks it as float32 in its shared memory, and after a cluster barrier every CTA sums one
// row slice of the tile over the S CTAs through distributed shared memory (fixed order
// r = 0..S-1, so results are reproducible), applies the epilogue and stores bf16.  No global
// scratch, one launch, and each CTA reads only 1/S of A.

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}

__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void cluster_arrive() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
}
__device__ __forceinline__ void cluster_wait() {
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// Address of this CTA's shared-memory location `local_smem_addr` as seen in CTA `cta` of the cluster.
__device__ __forceinline__ uint32_t dsmem_addr(uint32_t local_smem_addr, uint32_t cta) {
  uint32_t remote;
  asm("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_smem_addr), "r"(cta));
  return remote;
}

// Plain (schedulable) distributed-shared-memory load; ordering against the writers comes from
// the cluster barrier that precedes the reads.
__device__ __forceinline__ float4 ld_dsmem_f4(uint32_t remote_addr) {
  float4 v;
  asm("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];"
      : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
      : "r"(remote_addr));
  return v;
}

constexpr int kSiteSkProducer = 5, kSiteSkMma = 6, kSiteSkEpilogue = 7;

template <int BN>
struct SplitKCfg {
  static constexpr int kStageBytes = kBM * kBKBytes + BN * kBKBytes;
  static constexpr int kStages = (192 * 1024) / kStageBytes > 12 ? 12 : (192 * 1024) / kStageBytes;
  static constexpr int kRowFloats = BN + 4;  // padded row: conflict-free float4 access by row
  static constexpr int kStagingBytes = kBM * kRowFloats * 4;
  static constexpr int kPipeBytes = kStages * kStageBytes;
  static constexpr int kSmemBytes = (kPipeBytes > kStagingBytes ? kPipeBytes : kStagingBytes) + 1024 + 256;
  static constexpr int kTmemCols = BN < 32 ? 32 : BN;
};

// One work item of the split-K epilogue: f = the K-reduced accumulators of 8 consecutive columns
// of row m; multipliers and bias come from shared memory.
__device__ __forceinline__ void splitk_finish_item(const GemmParams& p, float (&f)[8], const uint4 rv, float rm,
                                                   const float* cm, const float* bias, int m, int n) {
#pragma unroll
  for (int j = 0; j < 8; ++j) f[j] = fmaf(f[j] * rm, cm[j], bias[j]);
  if (p.residual) {
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
    const uint32_t lo16 = __bfloat16_as_ushort(__float2bfloat16_rn(f[2 * j]));
    const uint32_t hi16 = __bfloat16_as_ushort(__float2bfloat16_rn(f[2 * j + 1]));
    ow[j] = lo16 | (hi16 << 16);
  }
  if (p.push_world > 0) {
#pragma unroll
    for (int r = 0; r < 8; ++r)
      if (r < p.push_world) *reinterpret_cast<uint4*>(p.push_out[r] + (long long)m * p.ldo + n) = o;
  } else {
    *reinterpret_cast<uint4*>(p.out + (long long)m * p.ldo + n) = o;
  }
}

template <int BN, bool IS_FP8>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_splitk_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                   const GemmParams p, const int S) {
  using Cfg = SplitKCfg<BN>;
  constexpr int kStages = Cfg::kStages;
  constexpr int kElemBytes = IS_FP8 ? 1 : 2;
  constexpr int kBKElems = kBKBytes / kElemBytes;
  constexpr uint32_t kIdesc = umma_idesc(IS_FP8 ? kFmtE4M3 : kFmtBF16, IS_FP8 ? kFmtE4M3 : kFmtBF16, 0, 0, kBM, BN);

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* smem_a = smem;
  uint8_t* smem_b = smem + kStages * kBM * kBKBytes;
  float* staging = reinterpret_cast<float*>(smem);  // reused once the main loop has drained
  constexpr int kBarOff = Cfg::kPipeBytes > Cfg::kStagingBytes ? Cfg::kPipeBytes : Cfg::kStagingBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kBarOff);
  uint64_t* full = bars;
  uint64_t* empty = bars + kStages;
  uint64_t* acc_full = bars + 2 * kStages;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_full + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int r = (int)cluster_ctarank();
  const int tile_n = blockIdx.x / S;
  const int n0 = tile_n * BN;
  // K blocks of this CTA: an even split of num_k_blocks over the S ranks
  const int kb0 = (int)((long long)p.num_k_blocks * r / S);
  const int kb1 = (int)((long long)p.num_k_blocks * (r + 1) / S);
  const int nkb = kb1 - kb0;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(full + s, 1);
      mbar_init(empty + s, 1);
    }
    mbar_init(acc_full, 1);
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
  pdl_trigger();  // tensor memory is allocated: the next kernel may be scheduled
  if (threadIdx.x != 0) pdl_wait();

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      int kk = nkb > 0 ? kb0 + (tile_n * 3) % nkb : kb0;  // staggered start, see gemm_tc_kernel
      {  // B of the first K blocks -> L2, ahead of the wait on the previous kernel (GemmParams::prefetch_l2)
        int k2 = kk;
        const int n_l2 = min(nkb, p.prefetch_l2);
        for (int i = 0; i < n_l2; ++i) {
          tma_prefetch_l2_2d(&tmap_b, k2 * kBKElems, n0);
          if (++k2 == kb1) k2 = kb0;
        }
      }
      pdl_wait();
      for (int i = 0; i < nkb; ++i) {
        // (the first trip round the ring finds every stage free: no barrier to test)
        if (i >= kStages &&
            !mbar_wait(empty + stage, phase ^ 1, abort_flag, p.d_status, XAXB_DEVICE_TIMEOUT * 1000 + kSiteSkProducer))
          break;
        mbar_arrive_expect_tx(full + stage, Cfg::kStageBytes);
        tma_load_2d(smem_a + stage * kBM * kBKBytes, &tmap_a, full + stage, kk * kBKElems, 0);
        tma_load_2d(smem_b + stage * BN * kBKBytes, &tmap_b, full + stage, kk * kBKElems, n0);
        if (++kk == kb1) kk = kb0;
        if (++stage == kStages) stage = 0, phase ^= 1;
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int i = 0; i < nkb; ++i) {
        ok = mbar_wait(full + stage, phase, abort_flag, p.d_status, XAXB_DEVICE_TIMEOUT * 1000 + kSiteSkMma);
        if (!ok) break;
        tc_fence_after_sync();
        const uint64_t a_desc = umma_desc_kmajor_sw128(smem_u32(smem_a + stage * kBM * kBKBytes));
        const uint64_t b_desc = umma_desc_kmajor_sw128(smem_u32(smem_b + stage * BN * kBKBytes));
#pragma unroll
        for (int k = 0; k < kBKBytes / 32; ++k) {
          if (IS_FP8)
            umma_f8(tmem_base, a_desc + 2 * k, b_desc + 2 * k, kIdesc | p.idesc_or, (i | k) != 0);
          else
            umma_f16(tmem_base, a_desc + 2 * k, b_desc + 2 * k, kIdesc, (i | k) != 0);
        }
        // a stage is handed back only if a later K block will use it: a commit costs this thread about as
        // much as an MMA, and a CTA's share of K is often no longer than the ring
        if (i + kStages < nkb) umma_commit(empty + stage);
        if (++stage == kStages) stage = 0, phase ^= 1;
      }
      if (ok) umma_commit(acc_full);  // with nkb == 0 this arrives at once: nothing was issued
    }
  }

  // ---- epilogue inputs, fetched while the main loop runs (the epilogue warps are idle until the
  // accumulator is complete): row multipliers of the tile's rows, column multipliers and bias of
  // its columns.  Reading them inside the reduction put a trip to L2 into every work item.
  __shared__ float s_rm[kBM], s_cm[BN], s_bias[BN];
  if (warp >= 2) {
    const int t = threadIdx.x - 64;
    {
      const int m = t;
      s_rm[t] = (p.row_mul && m < p.M) ? __ldg(p.row_mul + (long long)m * p.row_mul_stride) : 1.0f;
    }
    for (int j = t; j < BN; j += 128) {
      const int n = n0 + j;
      s_cm[j] = (p.col_mul && n < p.N) ? __ldg(p.col_mul + (long long)n * p.col_mul_stride) : 1.0f;
      s_bias[j] = (p.bias && n < p.N) ? __bfloat162float(p.bias[n]) : 0.0f;
    }
  }

  // ---- park the partial accumulator in shared memory (epilogue warps) ------------------------
  const int quarter = warp & 3;
  const int row = quarter * 32 + lane;
  bool ok = true;
  if (warp >= 2) {
    ok = mbar_wait(acc_full, 0, abort_flag, p.d_status, XAXB_DEVICE_TIMEOUT * 1000 + kSiteSkEpilogue);
    ok = __all_sync(0xffffffffu, ok);
    if (ok) {
      tc_fence_after_sync();
      const uint32_t taddr = tmem_base + (uint32_t(quarter * 32) << 16);
      float* srow = staging + row * Cfg::kRowFloats;
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += 32) {
        uint32_t v[32];
        if (nkb > 0) {
          tmem_ld_x32(taddr + c0, v);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = 0u;
        }
#pragma unroll
        for (int i = 0; i < 32; i += 4)
          *reinterpret_cast<float4*>(srow + c0 + i) = make_float4(__uint_as_float(v[i]), __uint_as_float(v[i + 1]),
                                                                  __uint_as_float(v[i + 2]), __uint_as_float(v[i + 3]));
      }
    }
    tc_fence_before_sync();
  }
  __syncwarp();
  cluster_sync_all();  // every CTA's partial tile is visible cluster-wide

  // ---- reduce this CTA's row slice over the S ranks, epilogue, store ---------------------------
  // CTA r owns rows [r * 128/S, (r+1) * 128/S) of the tile.  Work item = (row, 8 consecutive
  // columns), consecutive threads take consecutive column groups of a row, so shared-memory
  // reads (local and remote), the residual read and the bf16 store are all contiguous.  A thread
  // first sums its items over the ranks (all its remote reads), then the CTA tells the cluster it
  // is done reading -- so the peers' exit does not wait for this CTA's stores -- and only then
  // applies multipliers, bias and residual and stores.
  constexpr int kGroups = BN / 8;
  constexpr int kMaxItems = 8;  // per thread: rows_per * kGroups / 128
  const int rows_per = kBM / S;
  const int n_items = rows_per * kGroups;
  const bool fast = n_items <= kMaxItems * 128;
  float fsum[kMaxItems][8];
  uint4 resv[kMaxItems];
  if (warp >= 2 && ok) {
    const int t = threadIdx.x - 64;          // 0..127
    uint32_t peer[8];
#pragma unroll
    for (int src = 0; src < 8; ++src) peer[src] = dsmem_addr(smem_u32(staging), (uint32_t)(src < S ? src : 0));
    if (fast) {
#pragma unroll
      for (int k = 0; k < kMaxItems; ++k) {
        const int it = t + k * 128;
        resv[k] = make_uint4(0, 0, 0, 0);
        if (it < n_items && p.residual) {
          const int m = r * rows_per + it / kGroups, n = n0 + (it % kGroups) * 8;
          if (m < p.M && n < p.N) resv[k] = *reinterpret_cast<const uint4*>(p.residual + (long long)m * p.ldr + n);
        }
      }
#pragma unroll
      for (int k = 0; k < kMaxItems; ++k) {
        const int it = t + k * 128;
#pragma unroll
        for (int j = 0; j < 8; ++j) fsum[k][j] = 0.0f;
        if (it < n_items) {
          const int m = r * rows_per + it / kGroups, g8 = it % kGroups;
          const uint32_t off = (uint32_t)(m * Cfg::kRowFloats + g8 * 8) * 4u;
          float4 lo[8], hi[8];
#pragma unroll
          for (int src = 0; src < 8; ++src) {
            if (src < S) {
              lo[src] = ld_dsmem_f4(peer[src] + off);
              hi[src] = ld_dsmem_f4(peer[src] + off + 16);
            }
          }
#pragma unroll
          for (int src = 0; src < 8; ++src) {
            if (src < S) {
              fsum[k][0] += lo[src].x, fsum[k][1] += lo[src].y, fsum[k][2] += lo[src].z, fsum[k][3] += lo[src].w;
              fsum[k][4] += hi[src].x, fsum[k][5] += hi[src].y, fsum[k][6] += hi[src].z, fsum[k][7] += hi[src].w;
            }
          }
        }
      }
    } else {
      for (int it = t; it < n_items; it += 128) {
        const int m = r * rows_per + it / kGroups;
        const int g8 = it % kGroups;
        const int n = n0 + g8 * 8;
        if (m >= p.M || n >= p.N) continue;
        const uint32_t off = (uint32_t)(m * Cfg::kRowFloats + g8 * 8) * 4u;
        uint4 rv = make_uint4(0, 0, 0, 0);
        if (p.residual) rv = *reinterpret_cast<const uint4*>(p.residual + (long long)m * p.ldr + n);
        float f[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#pragma unroll
        for (int src = 0; src < 8; ++src) {
          if (src < S) {
            const float4 lo = ld_dsmem_f4(peer[src] + off), hi = ld_dsmem_f4(peer[src] + off + 16);
            f[0] += lo.x, f[1] += lo.y, f[2] += lo.z, f[3] += lo.w;
            f[4] += hi.x, f[5] += hi.y, f[6] += hi.z, f[7] += hi.w;
          }
        }
        splitk_finish_item(p, f, rv, s_rm[m], s_cm + g8 * 8, s_bias + g8 * 8, m, n);
      }
    }
  }
  __syncwarp();
  cluster_arrive();  // this CTA has finished reading its peers' shared memory
  if (warp >= 2 && ok && fast) {
    const int t = threadIdx.x - 64;
#pragma unroll
    for (int k = 0; k < kMaxItems; ++k) {
      const int it = t + k * 128;
      if (it < n_items) {
        const int m = r * rows_per + it / kGroups, g8 = it % kGroups, n = n0 + g8 * 8;
        if (m < p.M && n < p.N) splitk_finish_item(p, fsum[k], resv[k], s_rm[m], s_cm + g8 * 8, s_bias + g8 * 8, m, n);
      }
    }
  }
  if (p.push_world > 0 && warp >= 2) {
    // Every epilogue thread's peer stores precede the barrier; one thread then makes them visible
    // system-wide (one fence) and tells every rank how many 16-byte pieces of its staging slot are
    // complete with relaxed adds: fence + relaxed add is a release, and it is paid once.  Releasing
    // adds instead (each one a fence of its own) cost 6.7 us more per GEMM on two GPUs.
    epilogue_sync();
    if (threadIdx.x == 64 && ok) {
      const int row0 = r * rows_per;
      const int rows_ok = max(0, min(p.M, row0 + rows_per) - row0);
      const int cols_ok = max(0, min(BN, p.N - n0));
      const unsigned int pieces = (unsigned int)(rows_ok * (cols_ok / 8));
      __threadfence_system();
#pragma unroll
      for (int dst = 0; dst < 8; ++dst)
        if (dst < p.push_world)
          asm volatile("red.relaxed.sys.global.add.u32 [%0], %1;" ::"l"(p.push_flag[dst]), "r"(pieces) : "memory");
    }
  }
  __syncwarp();
  cluster_wait();  // the peers have finished reading this CTA's shared memory
  __syncthreads();
  if (warp == 2) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, Cfg::kTmemCols);
  }
}

template <int BN, bool IS_FP8>
static int launch_splitk(const Ctx* ctx, cudaStream_t stream, const void* a, long long lda_bytes, const void* b,
                         long long ldb_bytes, GemmParams& p, int S) {
  using Cfg = SplitKCfg<BN>;
  constexpr int kElemBytes = IS_FP8 ? 1 : 2;
  CUtensorMap ta, tb;
  int rc = make_tmap_2d(ctx, &ta, a, kElemBytes, (uint64_t)p.K, (uint64_t)p.M, (uint64_t)lda_bytes,
                        kBKBytes / kElemBytes, kBM);
  if (rc) return rc;
  rc = make_tmap_2d(ctx, &tb, b, kElemBytes, (uint64_t)p.K, (uint64_t)p.N, (uint64_t)ldb_bytes, kBKBytes / kElemBytes,
                    BN);
  if (rc) return rc;
  p.tiles_m = 1;
  p.tiles_n = (p.N + BN - 1) / BN;
  p.num_k_blocks = (int)(((long long)p.K * kElemBytes + kBKBytes - 1) / kBKBytes);
  rc = ensure_dynamic_smem<gemm_splitk_kernel<BN, IS_FP8>>(ctx, Cfg::kSmemBytes, "gemm_splitk_kernel");
  if (rc) return rc;
  cudaError_t e = launch_kernel(gemm_splitk_kernel<BN, IS_FP8>, dim3((unsigned)(p.tiles_n * S), 1, 1), dim3(kGemmThreads),
                                Cfg::kSmemBytes, stream, (unsigned)S, ta, tb, p, S);
  if (e != cudaSuccess) {
    set_last_error("gemm_splitk_kernel launch: %s", cudaGetErrorString(e));
    return XAXB_LAUNCH_FAILED;
  }
  return check_launch("gemm_splitk_kernel");
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
  CUtensorMap tout;
  if (Cfg::kTmaStore) {
    rc = make_tmap_2d(ctx, &tout, p.out, 2, (uint64_t)p.N, (uint64_t)p.M, (uint64_t)p.ldo * 2, 64, kBM);
    if (rc) return rc;
  } else {
    tout = ta;  // unused by the direct-store epilogue
  }
  p.tiles_m = (p.M + kBM - 1) / kBM;
  p.tiles_n = (p.N + BN - 1) / BN;
  p.num_k_blocks = (int)(((long long)p.K * kElemBytes + kBKBytes - 1) / kBKBytes);
  rc = ensure_dynamic_smem<gemm_tc_kernel<BN, IS_FP8>>(ctx, Cfg::kSmemBytes, "gemm_tc_kernel");
  if (rc) return rc;
  const int tiles = p.tiles_m * p.tiles_n;
  const int grid = tiles < ctx->num_sms ? tiles : ctx->num_sms;
  launch_kernel(gemm_tc_kernel<BN, IS_FP8>, grid, dim3(kGemmThreads), Cfg::kSmemBytes, stream, 1, ta, tb, tout, p);
  return check_launch("gemm_tc_kernel");
}

}  // namespace xaxb

#include "gemm_2cta.cuh"

namespace xaxb {

// Tile width (and, for M <= 128, the split-K factor) from a small cost model: a CTA ingests
// operand bytes at a bounded rate, the GPU as a whole at HBM rate, and the tensor core has its
// own rate.  Narrow tiles give more CTAs but re-read A once per N tile; splitting K gives more
// CTAs without that cost, at the price of a cluster-wide reduction.
struct GemmPlan {
  int bn;
  int split;
};

static int g_force_bn = 0, g_force_split = 0;  // test hook (xaxb_gemm_force_plan)
static int g_prefetch_l2 = kMaxPrefetchBlocks;  // xaxb_gemm_set_prefetch

// `one_wave_kernel`: every candidate runs on the split-K kernel (one tile per CTA, not persistent), as
// the pushing epilogue requires; a "split" of 1 is then a plain tile per CTA, in as many waves as needed.
static GemmPlan pick_plan(long long M, long long N, long long K, int elem_bytes, int num_sms,
                          bool one_wave_kernel = false) {
  // Fitted to measurements on B200 (decode shapes, weights streamed from HBM): a CTA whose
  // shared memory is all load stages ingests ~60 GB/s (in-flight bytes / loaded latency); a
  // launch has ~2.4 us of fixed time; every further wave of tiles on the persistent kernel
  // ~2 us; a cluster reduction 1.8 us (2 CTAs) or 3.9 us (4 CTAs) plus 0.02 us per tile column.
  // Clusters of 8 schedule poorly next to ~200 KB of shared memory per CTA and are not used;
  // split-K is only used when all its CTAs are resident at once.
  const long long tiles_m = (M + kBM - 1) / kBM;
  const double rows_a = (double)(M < kBM ? M : kBM);
  const double r_sm = 60e9, r_hbm = 6.0e12, r_mma = (elem_bytes == 1 ? 4.5e15 : 2.25e15) / 148.0 * 0.75;
  const long long nkb = (K * elem_bytes + kBKBytes - 1) / kBKBytes;
  const int cand[4] = {256, 128, 64, 32};
  GemmPlan best = {32, 1};
  double best_t = 1e30;
  for (int i = 0; i < 4; ++i) {
    const int bn = cand[i];
    if (bn > 32 && bn >= 2 * N) continue;
    for (int s = 1; s <= 4; s *= 2) {
      const long long ctas = tiles_m * ((N + bn - 1) / bn) * s;
      if (s > 1 && (tiles_m != 1 || nkb < 2 * s || ctas > num_sms)) continue;
      const double waves = (double)((ctas + num_sms - 1) / num_sms);
      const double t_sm = waves * (rows_a + bn) * (double)K / s * elem_bytes / r_sm;
      const double t_mma = waves * 2.0 * kBM * bn * (double)K / s / r_mma;
      const double t_hbm = (double)(N + M) * K * elem_bytes / r_hbm;
      double t = t_sm > t_mma ? t_sm : t_mma;
      if (t_hbm > t) t = t_hbm;
      t += 2.4e-6 + (waves - 1) * 2e-6;
      if (s > 1) t += (s == 2 ? 1.8e-6 : 3.9e-6) + 0.02e-6 * bn;
      if (one_wave_kernel && s == 1) t += 0.8e-6;  // the tile still goes through shared memory once
      if (bn == 32) t += 3e-6;  // measured: 32-wide tiles pay ~3 us more than their byte count says
      if (t < best_t) best_t = t, best = {bn, s};
    }
  }
  if (g_force_bn && g_force_bn < 384) best.bn = g_force_bn;
  if (g_force_split) best.split = g_force_split;
  return best;
}

// Where a tensor-parallel GEMM pushes its output (see GemmParams::push_out).
struct PushTarget {
  void* const* peer_bases;
  int rank, world;
  int64_t slot_offset_bytes;  // of this rank's slot inside every rank's buffer
  int64_t flag_offset_bytes;  // of the arrival counter inside every rank's buffer
};

template <bool IS_FP8>
static int gemm_entry(xaxb_ctx* ctx_, void* stream, const void* a, int64_t lda, const void* b, int64_t ldb, int64_t M,
                      int64_t N, int64_t K, const float* row_mul, int row_mul_stride, const float* col_mul,
                      int col_mul_stride, const void* bias, const void* residual, int64_t ldr, void* out,
                      int64_t ldo, const PushTarget* push = nullptr, uint32_t idesc_or = 0) {
  if (push) {
    if (!push->peer_bases || push->world < 1 || push->world > 8 || push->rank < 0 || push->rank >= push->world ||
        (push->slot_offset_bytes & 15) || (push->flag_offset_bytes & 3) || push->slot_offset_bytes < 0 ||
        push->flag_offset_bytes < 0 || M > kBM) {
      set_last_error("gemm push: needs 1 <= world <= 8, 0 <= rank < world, aligned offsets and M <= %d", kBM);
      return XAXB_BAD_ARGUMENT;
    }
    for (int r = 0; r < push->world; ++r)
      if (!push->peer_bases[r] || (reinterpret_cast<uintptr_t>(push->peer_bases[r]) & 15)) {
        set_last_error("gemm push: mapping of rank %d is null or not 16-byte aligned", r);
        return XAXB_BAD_ARGUMENT;
      }
    out = static_cast<uint8_t*>(push->peer_bases[push->rank]) + push->slot_offset_bytes;  // for the argument checks
    ldo = N;
  }
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
  p.idesc_or = idesc_or;
  p.d_status = ctx->d_status;
  p.prefetch_l2 = pdl_enabled() ? g_prefetch_l2 : 0;
  p.push_world = 0;
  p.ce_part = nullptr;
  p.ce_targets = nullptr;
  for (int r = 0; r < 8; ++r) p.push_out[r] = nullptr, p.push_flag[r] = nullptr;
  if (push) {
    p.push_world = push->world;
    for (int r = 0; r < push->world; ++r) {
      uint8_t* base = static_cast<uint8_t*>(push->peer_bases[r]);
      p.push_out[r] = reinterpret_cast<__nv_bfloat16*>(base + push->slot_offset_bytes);
      p.push_flag[r] = reinterpret_cast<unsigned int*>(base + push->flag_offset_bytes);
    }
  }
  p.band = 32;  // measured best for 128-row tiles at 8192^3 (2, 4, 8, 16, 32 tried); 16 for the pair kernel
  if (const char* e = getenv("XAXB_GEMM_BAND")) p.band = atoi(e) > 0 ? atoi(e) : 32;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  GemmPlan plan = pick_plan(M, N, K, eb, ctx->num_sms, push != nullptr);
  // Large problems go to the CTA-pair kernel: 256 x 256 tiles need a third less operand traffic
  // per SM, which is what bounds the single-CTA kernel.  It wants at least one full round of tiles
  // for the pairs (measured on the prefill shapes of configs 2 and 5 and on config 1: equal or faster
  // than 128 x 256 tiles from 128 pair tiles up, e.g. 95 against 104 us for 2048 x 4096 x 14336).
  const bool pair_ok = M > kBM && N >= 256;
  const long long pair_tiles = ((long long)(M + 255) / 256) * ((N + 255) / 256);
  const bool force_pair = g_force_bn == 512 || g_force_bn == 448 || g_force_bn == 384;  // 2 x the tile width
  if (!push && ((force_pair && pair_ok) ||
                (g_force_bn == 0 && pair_ok && plan.bn == 256 && plan.split == 1 && 2 * pair_tiles >= ctx->num_sms)))
    return launch_gemm_2cta<IS_FP8>(ctx, s, a, lda * eb, b, ldb * eb, p, force_pair ? g_force_bn / 2 : 0);
  if (plan.split > 1 || push) {  // the pushing epilogue lives in the split-K kernel (a "split" of 1 included)
    if (plan.bn == 512) plan.bn = 256;
    if (M > kBM || plan.split > 8) {
      set_last_error("gemm: split-K plan (bn=%d, split=%d) is invalid for M=%lld", plan.bn, plan.split, (long long)M);
      return XAXB_BAD_ARGUMENT;
    }
    switch (plan.bn) {
      case 256: return launch_splitk<256, IS_FP8>(ctx, s, a, lda * eb, b, ldb * eb, p, plan.split);
      case 128: return launch_splitk<128, IS_FP8>(ctx, s, a, lda * eb, b, ldb * eb, p, plan.split);
      case 64: return launch_splitk<64, IS_FP8>(ctx, s, a, lda * eb, b, ldb * eb, p, plan.split);
      default: return launch_splitk<32, IS_FP8>(ctx, s, a, lda * eb, b, ldb * eb, p, plan.split);
    }
  }
  switch (plan.bn) {
    case 256: return launch_gemm<256, IS_FP8>(ctx, s, a, lda * eb, b, ldb * eb, p);
    case 128: return launch_gemm<128, IS_FP8>(ctx, s, a, lda * eb, b, ldb * eb, p);
    case 64: return launch_gemm<64, IS_FP8>(ctx, s, a, lda * eb, b, ldb * eb, p);
    default: return launch_gemm<32, IS_FP8>(ctx, s, a, lda * eb, b, ldb * eb, p);
  }
}

}  // namespace xaxb

using namespace xaxb;

extern "C" {

int xaxb_gemm_force_plan(int bn, int split) {
  if ((bn != 0 && bn != 32 && bn != 64 && bn != 128 && bn != 256 && bn != 512 && bn != 448 && bn != 384) ||
      (split != 0 && split != 1 && split != 2 && split != 4 && split != 8))
    return XAXB_BAD_ARGUMENT;
  g_force_bn = bn;
  g_force_split = split;
  return XAXB_OK;
}

int xaxb_gemm_set_prefetch(int blocks_before_wait) {
  if (blocks_before_wait < 0 || blocks_before_wait > 4096) return XAXB_BAD_ARGUMENT;
  g_prefetch_l2 = blocks_before_wait;
  return XAXB_OK;
}

int xaxb_gemm_fp8_formats(xaxb_ctx* ctx, void* stream, const void* a_fp8, int64_t lda, int a_is_e5m2,
                          const void* b_fp8, int64_t ldb, int b_is_e5m2, int64_t M, int64_t N, int64_t K,
                          const float* row_mul, int row_mul_stride, const float* col_mul, int col_mul_stride,
                          const void* bias_bf16, const void* residual_bf16, int64_t ldr, void* out_bf16, int64_t ldo) {
  const uint32_t idesc_or = (a_is_e5m2 ? 1u << 7 : 0u) | (b_is_e5m2 ? 1u << 10 : 0u);
  return gemm_entry<true>(ctx, stream, a_fp8, lda, b_fp8, ldb, M, N, K, row_mul, row_mul_stride, col_mul,
                          col_mul_stride, bias_bf16, residual_bf16, ldr, out_bf16, ldo, nullptr, idesc_or);
}

int xaxb_gemm_fp8(xaxb_ctx* ctx, void* stream, const void* a_e4m3, int64_t lda, const void* b_e4m3, int64_t ldb,
                  int64_t M, int64_t N, int64_t K, const float* row_mul, int row_mul_stride, const float* col_mul,
                  int col_mul_stride, const void* bias_bf16, const void* residual_bf16, int64_t ldr, void* out_bf16,
                  int64_t ldo) {
  return gemm_entry<true>(ctx, stream, a_e4m3, lda, b_e4m3, ldb, M, N, K, row_mul, row_mul_stride, col_mul,
                          col_mul_stride, bias_bf16, residual_bf16, ldr, out_bf16, ldo);
}

int xaxb_gemm_fp8_push(xaxb_ctx* ctx, void* stream, const void* a_e4m3, int64_t lda, const void* b_e4m3, int64_t ldb,
                       int64_t M, int64_t N, int64_t K, const float* row_mul, int row_mul_stride, const float* col_mul,
                       int col_mul_stride, const void* bias_bf16, const void* residual_bf16, int64_t ldr,
                       void* const* peer_bases, int rank, int world, int64_t slot_offset_bytes,
                       int64_t flag_offset_bytes) {
  const PushTarget push = {peer_bases, rank, world, slot_offset_bytes, flag_offset_bytes};
  return gemm_entry<true>(ctx, stream, a_e4m3, lda, b_e4m3, ldb, M, N, K, row_mul, row_mul_stride, col_mul,
                          col_mul_stride, bias_bf16, residual_bf16, ldr, nullptr, 0, &push);
}

int xaxb_gemm_bf16(xaxb_ctx* ctx, void* stream, const void* a_bf16, int64_t lda, const void* b_bf16, int64_t ldb,
                   int64_t M, int64_t N, int64_t K, const float* row_mul, int row_mul_stride, const float* col_mul,
                   int col_mul_stride, const void* bias_bf16, const void* residual_bf16, int64_t ldr, void* out_bf16,
                   int64_t ldo) {
  return gemm_entry<false>(ctx, stream, a_bf16, lda, b_bf16, ldb, M, N, K, row_mul, row_mul_stride, col_mul,
                           col_mul_stride, bias_bf16, residual_bf16, ldr, out_bf16, ldo);
}

}  // extern "C"

// ---------------------------------------------------------------------------------------
// lm_head + cross-entropy / accuracy without materialising the logits
// (xax/arch/llm.py:718-887: chunked_cross_entropy_loss / chunked_cross_entropy_acc, forward).

namespace xaxb {

constexpr int kCeTile = 256;  // vocabulary columns per partial result

// One warp per row: merges the row's per-tile (max, sum, target logit, arg-max) in tile order.
// loss = logsumexp(logits) - logit[target]; pred = first index of the maximum.
__global__ void __launch_bounds__(256) ce_merge_kernel(const float4* __restrict__ part, int tiles_n, int T,
                                                       float* __restrict__ row_loss, int32_t* __restrict__ row_pred) {
  pdl_trigger();
  pdl_wait();
  const int row = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (row >= T) return;
  float m = -INFINITY, l = 0.0f, tv = -INFINITY;
  int best = 0x7fffffff;
  for (int t = lane; t < tiles_n; t += 32) {
    const float4 v = part[(long long)row * tiles_n + t];
    const int idx = __float_as_int(v.w);
    if (v.x > m || (v.x == m && idx < best)) best = idx;  // tiles ascend, so do their columns
    const float mn = fmaxf(m, v.x);
    l = l * expf(m - mn) + v.y * expf(v.x - mn);
    m = mn;
    tv = fmaxf(tv, v.z);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float m2 = __shfl_xor_sync(0xffffffffu, m, o), l2 = __shfl_xor_sync(0xffffffffu, l, o);
    const float t2 = __shfl_xor_sync(0xffffffffu, tv, o);
    const int b2 = __shfl_xor_sync(0xffffffffu, best, o);
    if (m2 > m || (m2 == m && b2 < best)) best = b2;
    const float mn = fmaxf(m, m2);
    // (both sides -inf only when a lane had no tile: its l is 0 and exp(-inf - -inf) is never formed)
    const float a = m == -INFINITY ? 0.0f : l * expf(m - mn), b = m2 == -INFINITY ? 0.0f : l2 * expf(m2 - mn);
    l = a + b;
    m = mn;
    tv = fmaxf(tv, t2);
  }
  if (lane == 0) {
    if (row_loss) row_loss[row] = (m + logf(l)) - tv;
    if (row_pred) row_pred[row] = best;
  }
}

// Masked means over the rows, one CTA, fixed summation order: result = {mean loss, accuracy, count}.
__global__ void __launch_bounds__(1024) ce_finish_kernel(const float* __restrict__ row_loss,
                                                         const int32_t* __restrict__ row_pred,
                                                         const int32_t* __restrict__ targets,
                                                         const uint8_t* __restrict__ mask, int T, float* result) {
  pdl_trigger();
  pdl_wait();
  __shared__ float s_loss[1024], s_hit[1024], s_cnt[1024];
  float a = 0.0f, h = 0.0f, c = 0.0f;
  for (int i = threadIdx.x; i < T; i += 1024) {
    if (mask && !mask[i]) continue;
    a += row_loss[i];
    h += row_pred[i] == targets[i] ? 1.0f : 0.0f;
    c += 1.0f;
  }
  s_loss[threadIdx.x] = a, s_hit[threadIdx.x] = h, s_cnt[threadIdx.x] = c;
  __syncthreads();
  for (int o = 512; o > 0; o >>= 1) {
    if ((int)threadIdx.x < o) {
      s_loss[threadIdx.x] += s_loss[threadIdx.x + o];
      s_hit[threadIdx.x] += s_hit[threadIdx.x + o];
      s_cnt[threadIdx.x] += s_cnt[threadIdx.x + o];
    }
    __syncthreads();
  }
  if (threadIdx.x == 0) {
    const float n = s_cnt[0];
    result[0] = n > 0.0f ? s_loss[0] / n : 0.0f;  // :788 / :887: no valid position -> 0
    result[1] = n > 0.0f ? s_hit[0] / n : 0.0f;
    result[2] = n;
  }
}

}  // namespace xaxb

extern "C" int64_t xaxb_lm_head_cross_entropy_workspace_bytes(int64_t T, int64_t V) {
  if (T <= 0 || V <= 0) return 0;
  return T * ((V + kCeTile - 1) / kCeTile) * (int64_t)sizeof(float4);
}

extern "C" int xaxb_lm_head_cross_entropy(xaxb_ctx* ctx_, void* stream, const void* hidden_bf16, int64_t ldh,
                                          const void* weight_bf16, int64_t ldw, int64_t T, int64_t V, int64_t H,
                                          const int32_t* targets, const uint8_t* mask, void* workspace,
                                          int64_t workspace_bytes, float* row_loss, int32_t* row_pred, float* result) {
  if (!ctx_ || !hidden_bf16 || !weight_bf16 || !targets || !workspace || !row_loss || !row_pred || !result || T <= 0 ||
      V <= 0 || H <= 0) {
    set_last_error("lm_head_cross_entropy: null pointer or non-positive shape");
    return XAXB_BAD_ARGUMENT;
  }
  if ((H * 2) % 16 != 0 || T > 0x7fffffff || V > 0x7fffffff || (reinterpret_cast<uintptr_t>(workspace) & 15)) {
    set_last_error("lm_head_cross_entropy: hidden size %lld must be a multiple of 8 and the workspace 16-byte aligned",
                   (long long)H);
    return XAXB_BAD_ARGUMENT;
  }
  if (workspace_bytes < xaxb_lm_head_cross_entropy_workspace_bytes(T, V)) return XAXB_WORKSPACE_TOO_SMALL;
  const Ctx* ctx = reinterpret_cast<const Ctx*>(ctx_);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  GemmParams p;
  p.M = (int)T, p.N = (int)V, p.K = (int)H;
  p.row_mul = nullptr, p.row_mul_stride = 0, p.col_mul = nullptr, p.col_mul_stride = 0;
  p.bias = nullptr, p.residual = nullptr, p.ldr = 0;
  // never stored to: the store's tensor map only needs an aligned base and a row stride that is a multiple of 16 bytes
  p.out = static_cast<__nv_bfloat16*>(workspace);
  p.ldo = (V + 7) / 8 * 8;
  p.d_status = ctx->d_status;
  p.idesc_or = 0;
  p.prefetch_l2 = pdl_enabled() ? g_prefetch_l2 : 0;
  p.band = 32;
  p.push_world = 0;
  for (int r = 0; r < 8; ++r) p.push_out[r] = nullptr, p.push_flag[r] = nullptr;
  p.ce_part = static_cast<float4*>(workspace);
  p.ce_targets = targets;
  int rc = launch_gemm<kCeTile, false>(ctx, s, hidden_bf16, ldh * 2, weight_bf16, ldw * 2, p);
  if (rc) return rc;
  const int tiles_n = (int)((V + kCeTile - 1) / kCeTile);
  launch_kernel(ce_merge_kernel, dim3((unsigned)((T + 7) / 8)), dim3(256), 0, s, 1, static_cast<const float4*>(workspace),
                tiles_n, (int)T, row_loss, row_pred);
  rc = check_launch("ce_merge_kernel");
  if (rc) return rc;
  launch_kernel(ce_finish_kernel, dim3(1), dim3(1024), 0, s, 1, static_cast<const float*>(row_loss),
                static_cast<const int32_t*>(row_pred), targets, mask, (int)T, result);
  return check_launch("ce_finish_kernel");
}
