// Kernel 2, large-problem variant: 256 x BN output tiles (BN = 256, 224 or 192) computed by PAIRS of CTAs
// (a thread-block cluster of two SMs issuing tcgen05.mma.cta_group::2).
//
// The single-CTA kernel's 128 x 256 tile pulls 48 KiB of operands out of L2 for every
// 128 x 256 x 128-byte MMA block and is bound by the SM's L2 read port (~105 GB/s per SM
// measured), not by the tensor core.  With a CTA pair, CTA r loads rows [r*128, r*128+128) of
// the A tile and rows [r*128, r*128+128) of the B tile -- 32 KiB per CTA for the same MMA work
// per SM -- and one tcgen05.mma reads A and B halves from both CTAs' shared memory and writes
// each CTA's 128 accumulator rows into that CTA's tensor memory.  No multicast is involved: each
// CTA fetches its own halves with ordinary TMA tile loads.
//
// The narrower tiles exist for problems whose 256-wide tiles fill the last round of the persistent loop badly:
// 2048 x 8192 x 2048 is 256 tiles of 256 x 256, 3.46 rounds for 74 pairs and therefore four tile-times, but
// 296 tiles of 256 x 224, exactly four rounds of shorter tiles.  The launcher picks the width (see
// pick_pair_width).  224 columns are three 64-column output blocks and one of 32, which is stored
// through a second tensor map (32-column box, no swizzle).
//
// Synchronisation (leader = CTA rank 0 of the pair):
//   full[s]      in the leader, 2 arrivals (one arrive.expect_tx per CTA) + both CTAs' TMA bytes;
//   empty[s]     in each CTA; the leader's MMA thread commits to both (one local, one remote commit);
//   acc_full[b]  in each CTA; committed to both by the leader after the tile's last MMA;
//   acc_empty[b] in the leader, 8 arrivals (4 epilogue warps x 2 CTAs; the peer arrives remotely).
// Included by gemm_tc.cu (shares GemmParams, the planner and the epilogue helpers).
#pragma once

namespace xaxb {

constexpr int kSite2Producer = 31, kSite2Mma = 32, kSite2Epilogue = 33, kSite2MmaAcc = 34;

__device__ __forceinline__ void mbar_arrive_expect_tx_cluster(uint32_t cluster_addr, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cluster.b64 _, [%0], %1;" ::"r"(cluster_addr), "r"(bytes)
               : "memory");
}

__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}

// TMA tile load whose completion bytes are credited to a barrier that may live in the peer CTA.
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const CUtensorMap* map, uint32_t bar_cluster_addr, int x,
                                                 int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(map), "r"(bar_cluster_addr), "r"(x), "r"(y)
      : "memory");
}

__device__ __forceinline__ void umma_commit_pair(uint32_t bar_cluster_addr) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar_cluster_addr)
               : "memory");
}

template <bool IS_FP8>
__device__ __forceinline__ void umma_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                          uint32_t accumulate) {
  if (IS_FP8) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
  } else {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
  }
}

template <int BN_>
struct Gemm2Cfg {
  static_assert(BN_ % 32 == 0 && BN_ >= 128 && BN_ <= 256, "pair tile width");
  static constexpr int kBN = BN_;                       // columns per pair tile
  static constexpr int kBRows = BN_ / 2;                // rows of the B tile each CTA loads
  // A stage holds 256 bytes of K: two 128-byte swizzle spans ("boxes") per operand, eight MMAs.  What the
  // MMA thread spends per stage beyond the MMAs themselves (finding the stage's barrier complete, the
  // commits that free it: about a hundred cycles each, like an MMA) is then paid once per eight MMAs instead
  // of once per four; with 128-byte stages the thread needed ~650 cycles for four MMAs that keep the tensor
  // pipe busy for 512, and the pipe idled a fifth of the time.
  static constexpr int kBoxesPerStage = 2;
  static constexpr int kSlotBytes = kBoxesPerStage * kBM * kBKBytes;  // per CTA: a 32 KiB slot for A, one for B
  static constexpr int kStageBytes = 2 * kSlotBytes;
  static constexpr int kLoadBytes = kBoxesPerStage * (kBM + kBRows) * kBKBytes;  // what the loads of a stage deliver
  static constexpr int kAccStride = 256;                // columns between the two accumulators
  // Two staging blocks for the TMA stores: while the TMA unit reads one, the epilogue warps fill the other.
  // With a single block every 64-column store waited for the previous one's read, and a tile's epilogue
  // (four stores) took longer than the main loop of a short-K tile (config 1: K = 2048, 16 K blocks).
  // Five load stages of 32 KiB keep far more in flight than an SM's request capacity needs.
  static constexpr int kOutBlockBytes = kBM * 128;
  static constexpr int kEpiBytes = 2 * kOutBlockBytes + 2 * 256 * 4;
  static constexpr int kStages = 3;                     // 192 KiB of operands in flight
  static constexpr int kTmemCols = 512;                 // two 256-column accumulators
  static constexpr int kSmemBytes = kStages * kStageBytes + kEpiBytes + 256;  // (the array is declared 1024-aligned)
};

template <bool IS_FP8, int BN_>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_2cta_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                 const __grid_constant__ CUtensorMap tmap_out, const __grid_constant__ CUtensorMap tmap_out_half,
                 const GemmParams p) {
  pdl_wait();  // nothing below may run ahead of the previous kernel in the stream
  using Cfg = Gemm2Cfg<BN_>;
  constexpr int kStages = Cfg::kStages, BN = Cfg::kBN;
  constexpr int kElemBytes = IS_FP8 ? 1 : 2;
  constexpr int kBKElems = kBKBytes / kElemBytes;
  constexpr uint32_t kIdesc = umma_idesc(IS_FP8 ? kFmtE4M3 : kFmtBF16, IS_FP8 ? kFmtE4M3 : kFmtBF16, 0, 0, 2 * kBM, BN);

  extern __shared__ __align__(1024) uint8_t smem2[];   // swizzled tiles need 1024-byte alignment
  uint8_t* smem = smem2;
  uint8_t* smem_a = smem;                              // kStages x 32 KiB
  uint8_t* smem_b = smem + kStages * Cfg::kSlotBytes;  // kStages x 32 KiB
  uint8_t* stage_out = smem + kStages * Cfg::kStageBytes;
  float* cmul_s = reinterpret_cast<float*>(stage_out + 2 * Cfg::kOutBlockBytes);
  float* bias_s = cmul_s + 256;
  uint64_t* bars = reinterpret_cast<uint64_t*>(stage_out + Cfg::kEpiBytes);
  uint64_t* full = bars;
  uint64_t* empty = bars + kStages;
  uint64_t* acc_full = bars + 2 * kStages;
  uint64_t* acc_empty = acc_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();  // 0 = leader
  const int pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;
  const int num_tiles = p.tiles_m * p.tiles_n;  // 256 x BN tiles

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(full + s, 2);
      mbar_init(empty + s, 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(acc_full + i, 1);
      mbar_init(acc_empty + i, 8);
    }
    *abort_flag = 0;
    fence_mbar_init();
    prefetch_tmap(&tmap_a);
    prefetch_tmap(&tmap_b);
    prefetch_tmap(&tmap_out);
    if (BN % 64) prefetch_tmap(&tmap_out_half);
  }
  if (warp == 2) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                 "r"((uint32_t)Cfg::kTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  tc_fence_before_sync();
  __syncthreads();
  __syncwarp();
  cluster_sync_all();  // both CTAs' barriers exist before anyone signals across the pair
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  pdl_trigger();  // tensor memory is allocated: the next kernel may be scheduled

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer (both CTAs)
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = pair; tile < num_tiles && ok; tile += num_pairs) {
        int tm, tn;
        tile_coords(p.band, tile, p.tiles_m, p.tiles_n, tm, tn);
        const int m0 = tm * (2 * kBM) + (int)rank * kBM;
        const int n0 = tn * BN + (int)rank * Cfg::kBRows;
        int kk = (int)(((long long)tile * 5) % p.num_k_blocks);
        for (int kb = 0; kb < p.num_k_blocks; ++kb) {
          ok = mbar_wait(empty + stage, phase ^ 1, abort_flag, p.d_status, XAXB_DEVICE_TIMEOUT * 1000 + kSite2Producer);
          if (!ok) break;
          const uint32_t leader_full = dsmem_addr(smem_u32(full + stage), 0);
          mbar_arrive_expect_tx_cluster(leader_full, Cfg::kLoadBytes);
#pragma unroll
          for (int x = 0; x < Cfg::kBoxesPerStage; ++x) {
            const int k0 = (kk * Cfg::kBoxesPerStage + x) * kBKElems;  // (past K: zero fill)
            tma_load_2d_pair(smem_a + stage * Cfg::kSlotBytes + x * kBM * kBKBytes, &tmap_a, leader_full, k0, m0);
            tma_load_2d_pair(smem_b + stage * Cfg::kSlotBytes + x * Cfg::kBRows * kBKBytes, &tmap_b, leader_full, k0, n0);
          }
          if (++kk == p.num_k_blocks) kk = 0;
          if (++stage == kStages) stage = 0, phase ^= 1;
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (leader only)
    if (lane == 0 && rank == 0) {
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int tile = pair; tile < num_tiles && ok; tile += num_pairs) {
        ok = mbar_wait(acc_empty + acc, acc_phase ^ 1, abort_flag, p.d_status, XAXB_DEVICE_TIMEOUT * 1000 + kSite2MmaAcc);
        if (!ok) break;
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * Cfg::kAccStride;
        for (int kb = 0; kb < p.num_k_blocks; ++kb) {
          ok = mbar_wait(full + stage, phase, abort_flag, p.d_status, XAXB_DEVICE_TIMEOUT * 1000 + kSite2Mma);
          if (!ok) break;
          tc_fence_after_sync();
#pragma unroll
          for (int x = 0; x < Cfg::kBoxesPerStage; ++x) {
            const uint64_t a_desc = umma_desc_kmajor_sw128(smem_u32(smem_a + stage * Cfg::kSlotBytes + x * kBM * kBKBytes));
            const uint64_t b_desc =
                umma_desc_kmajor_sw128(smem_u32(smem_b + stage * Cfg::kSlotBytes + x * Cfg::kBRows * kBKBytes));
#pragma unroll
            for (int k = 0; k < kBKBytes / 32; ++k)
              umma_pair<IS_FP8>(d_tmem, a_desc + 2 * k, b_desc + 2 * k, kIdesc | p.idesc_or, (kb | x | k) != 0);
          }
          umma_commit_pair(smem_u32(empty + stage));
          umma_commit_pair(dsmem_addr(smem_u32(empty + stage), 1));
          if (++stage == kStages) stage = 0, phase ^= 1;
        }
        if (!ok) break;
        umma_commit_pair(smem_u32(acc_full + acc));
        umma_commit_pair(dsmem_addr(smem_u32(acc_full + acc), 1));
        if (++acc == 2) acc = 0, acc_phase ^= 1;
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (both CTAs)
    const int quarter = warp & 3;
    const int row_in_tile = quarter * 32 + lane;
    const int t = threadIdx.x - 64;
    int acc = 0;
    uint32_t acc_phase = 0;
    for (int tile = pair; tile < num_tiles; tile += num_pairs) {
      int tm, tn;
      tile_coords(p.band, tile, p.tiles_m, p.tiles_n, tm, tn);
      const int m0 = tm * (2 * kBM) + (int)rank * kBM;
      const int n0 = tn * BN;
      // The tile's multipliers and bias are fetched while its main loop is still running (every thread
      // passed the previous tile's last barrier after its last read of cmul_s / bias_s).
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
      bool ok = mbar_wait(acc_full + acc, acc_phase, abort_flag, p.d_status, XAXB_DEVICE_TIMEOUT * 1000 + kSite2Epilogue);
      if (!epilogue_all(ok)) break;  // (also publishes cmul_s / bias_s)
      tc_fence_after_sync();
      const uint32_t taddr = tmem_base + (uint32_t(quarter * 32) << 16) + acc * Cfg::kAccStride;
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += 64) {
        // the staging block about to be written was handed to the TMA unit two stores ago: that
        // store must have finished reading it (the one issued last may still be reading the other block)
        uint8_t* stage_blk = stage_out + ((c0 / 64) & 1) * Cfg::kOutBlockBytes;
        const bool half_blk = (BN % 64) != 0 && c0 + 64 > BN;  // the tile's last 32 columns: rows of 64 bytes, no swizzle
        if (t == 0) asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
        epilogue_sync();
#pragma unroll
        for (int h = 0; h < 64; h += 32) {
          if ((BN % 64) != 0 && c0 + h >= BN) break;
          uint32_t r[32];
          tmem_ld_x32(taddr + c0 + h, r);
          tmem_ld_wait();
          if (c0 + h + 32 >= BN) {  // accumulator read out: tell the leader's MMA thread
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(dsmem_addr(smem_u32(acc_empty + acc), 0));
          }
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            const int cc = c0 + h + v * 8;
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
            if (half_blk)
              *reinterpret_cast<uint4*>(stage_blk + row_in_tile * 64 + v * 16) = o;
            else
              *reinterpret_cast<uint4*>(stage_blk + sw128_offset(row_in_tile, (h + v * 8) / 8)) = o;
          }
        }
        fence_proxy_async_smem();
        epilogue_sync();
        if (t == 0) {
          if (n0 + c0 < p.N && m0 < p.M)
            asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
                         ::"l"(half_blk ? &tmap_out_half : &tmap_out), "r"(smem_u32(stage_blk)), "r"(n0 + c0), "r"(m0)
                         : "memory");
          // one group per block, stored or not, so that "all but the latest group" always means "the
          // store that used the other staging block"
          asm volatile("cp.async.bulk.commit_group;" ::: "memory");
        }
      }
      if (++acc == 2) acc = 0, acc_phase ^= 1;
    }
    if (t == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
  }

  // ---------------------------------------------------------------------- teardown
  tc_fence_before_sync();
  __syncthreads();
  __syncwarp();
  cluster_sync_all();  // no remote arrival or operand read can still target a CTA that leaves
  if (warp == 2) {
    tc_fence_after_sync();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)Cfg::kTmemCols)
                 : "memory");
  }
}

// How many CTA pairs can be resident at once.  Not every SM has a partner it can form a pair with, so the
// driver is asked instead of assuming num_sms / 2.  (All tile widths use the same shared memory and threads.)
template <bool IS_FP8>
static int max_resident_pairs(const Ctx* ctx) {
  static int max_pairs = 0;
  if (max_pairs == 0) {
    // the query fails for more than 48 KiB of dynamic shared memory unless the kernel has opted in
    if (ensure_dynamic_smem<gemm_2cta_kernel<IS_FP8, 256>>(ctx, Gemm2Cfg<256>::kSmemBytes, "gemm_2cta_kernel"))
      return ctx->num_sms / 2 - 8;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(2 * (ctx->num_sms / 2)), 1, 1);
    cfg.blockDim = dim3(kGemmThreads, 1, 1);
    cfg.dynamicSmemBytes = Gemm2Cfg<256>::kSmemBytes;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int n = 0;
    cudaError_t qe = cudaOccupancyMaxActiveClusters(&n, gemm_2cta_kernel<IS_FP8, 256>, &cfg);
    max_pairs = (qe == cudaSuccess && n > 0) ? n : ctx->num_sms / 2 - 8;
  }
  return max_pairs;
}

template <bool IS_FP8, int BN>
static int launch_gemm_2cta_bn(const Ctx* ctx, cudaStream_t stream, const void* a, long long lda_bytes, const void* b,
                               long long ldb_bytes, GemmParams& p, int max_pairs) {
  using Cfg = Gemm2Cfg<BN>;
  constexpr int kElemBytes = IS_FP8 ? 1 : 2;
  CUtensorMap ta, tb, tout, thalf;
  int rc = make_tmap_2d(ctx, &ta, a, kElemBytes, (uint64_t)p.K, (uint64_t)p.M, (uint64_t)lda_bytes,
                        kBKBytes / kElemBytes, kBM);
  if (rc) return rc;
  rc = make_tmap_2d(ctx, &tb, b, kElemBytes, (uint64_t)p.K, (uint64_t)p.N, (uint64_t)ldb_bytes, kBKBytes / kElemBytes,
                    Cfg::kBRows);
  if (rc) return rc;
  rc = make_tmap_2d(ctx, &tout, p.out, 2, (uint64_t)p.N, (uint64_t)p.M, (uint64_t)p.ldo * 2, 64, kBM);
  if (rc) return rc;
  if (BN % 64) {  // the tile's last 32 columns
    rc = make_tmap_2d_plain(ctx, &thalf, p.out, 2, (uint64_t)p.N, (uint64_t)p.M, (uint64_t)p.ldo * 2, 32, kBM);
    if (rc) return rc;
  } else {
    thalf = tout;  // never read
  }
  p.tiles_m = (p.M + 2 * kBM - 1) / (2 * kBM);
  if (!getenv("XAXB_GEMM_BAND")) p.band = 16;
  p.tiles_n = (p.N + BN - 1) / BN;
  constexpr int kStageKBytes = Cfg::kBoxesPerStage * kBKBytes;
  p.num_k_blocks = (int)(((long long)p.K * kElemBytes + kStageKBytes - 1) / kStageKBytes);
  if (int rc2 = ensure_dynamic_smem<gemm_2cta_kernel<IS_FP8, BN>>(ctx, Cfg::kSmemBytes, "gemm_2cta_kernel")) return rc2;
  const int tiles = p.tiles_m * p.tiles_n;
  // The kernel is persistent: every pair must be resident at once.
  const int pairs = tiles < max_pairs ? tiles : max_pairs;
  cudaError_t e = launch_kernel(gemm_2cta_kernel<IS_FP8, BN>, dim3((unsigned)(2 * pairs), 1, 1), dim3(kGemmThreads),
                                Cfg::kSmemBytes, stream, 2u, ta, tb, tout, thalf, p);
  if (e != cudaSuccess) {
    set_last_error("gemm_2cta_kernel launch: %s", cudaGetErrorString(e));
    return XAXB_LAUNCH_FAILED;
  }
  return check_launch("gemm_2cta_kernel");
}

// Width of the pair tiles: every pair walks ceil(tiles / pairs) tiles.  A tile's time follows the operand bytes
// its CTAs pull in per K block (128 rows of A plus width / 2 rows of B each), not its flops: measured per round,
// 224 columns cost 0.94 and 192 columns 0.86 of what 256 columns cost.  So the width with the smallest
// rounds x (256 + width + 32) wins; 256 unless a narrower one is at least 3 % cheaper (2048 x 8192 x 2048:
// 40.0 us with 224 columns against 42.0).  force_bn (256 / 224 / 192) overrides (tests).
static int pick_pair_width(long long M, long long N, int max_pairs, int force_bn) {
  if (force_bn) return force_bn;
  const long long tiles_m = (M + 2 * kBM - 1) / (2 * kBM);
  auto cost = [&](int bn) {
    const long long tiles = tiles_m * ((N + bn - 1) / bn);
    return ((tiles + max_pairs - 1) / max_pairs) * (long long)(256 + bn + 32);
  };
  int best = 256;
  long long best_cost = cost(256) * 97;  // in hundredths: a narrower tile must beat 97 % of this
  for (int bn : {224, 192}) {
    const long long c = cost(bn) * 100;
    if (c < best_cost) best = bn, best_cost = c;
  }
  return best;
}

template <bool IS_FP8>
static int launch_gemm_2cta(const Ctx* ctx, cudaStream_t stream, const void* a, long long lda_bytes, const void* b,
                            long long ldb_bytes, GemmParams& p, int force_bn) {
  const int max_pairs = max_resident_pairs<IS_FP8>(ctx);
  switch (pick_pair_width(p.M, p.N, max_pairs, force_bn)) {
    case 224: return launch_gemm_2cta_bn<IS_FP8, 224>(ctx, stream, a, lda_bytes, b, ldb_bytes, p, max_pairs);
    case 192: return launch_gemm_2cta_bn<IS_FP8, 192>(ctx, stream, a, lda_bytes, b, ldb_bytes, p, max_pairs);
    default: return launch_gemm_2cta_bn<IS_FP8, 256>(ctx, stream, a, lda_bytes, b, ldb_bytes, p, max_pairs);
  }
}

}  // namespace xaxb
