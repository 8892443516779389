// Kernel 3b: causal GQA prefill attention against the KV cache (flash-attention style, one
// pass, float32 online softmax), on tcgen05 tensor cores.
//
// One CTA = 128 consecutive queries of one (sequence, query head); 128 threads, thread r owns
// query row r.  Two CTAs share an SM (112 KB of shared memory and 256 TMEM columns each), so one CTA's
// tensor-core work runs under the other's softmax.  For every 64-token tile of the cache up to the
// diagonal:
//   S  = Q K^T      UMMA M = 128 queries, N = 64 tokens, K = D       (A = Q, B = K tile; K-major)
//   thread r reads row r of S from TMEM, applies the causal mask and the online-softmax
//   update, writes bf16 probabilities to shared memory (the reference also rounds the
//   probabilities to the value dtype before P.V),
//   PV = P V        UMMA M = 128 queries, N = D, K = 64 tokens       (A = P K-major, B = V tile
//                                                                     MN-major: D contiguous)
//   thread r reads row r of PV and folds it into its float32 output row: o = o * alpha + PV.
// K / V tiles arrive by TMA (128-byte swizzle) into a two-stage ring, so the next tile loads
// while the current one is processed.  Query position i of sequence b is positions[b] + i and
// sees cache rows 0 .. positions[b] + i.
#include "common.cuh"

namespace xaxb {

constexpr int kPfTile = 128;  // queries per CTA
constexpr int kPfKeys = 64;   // cache rows per K / V tile
constexpr int kSitePfKV = 21, kSitePfS = 22, kSitePfO = 23;

struct PrefillParams {
  const __nv_bfloat16* q;    // [B*T, Hq, D] rotated
  __nv_bfloat16* out;        // [B*T, Hq, D]
  const int32_t* positions;  // [B]
  int T, Hq, Hkv;
  float sm_scale;
  int window;  // sliding window: query at position q sees keys q - window .. q; < 0 = unlimited
  // cross-attention (xax/arch/attention.py:1176-1182, is_causal=False): positions[b] is the number of
  // context rows of sequence b and every query row sees all of them; only the length mask remains
  int cross;
  long long max_len;
  int* d_status;
};

template <int D>
struct PrefillSmem {
  static constexpr int kHalfBytes = kPfTile * 128;          // Q: 128 rows x 128 B per 64-element box
  static constexpr int kKVHalfBytes = kPfKeys * 128;        // K / V: 64 rows x 128 B per box
  static constexpr int kQBytes = kPfTile * D * 2;
  static constexpr int kKVBytes = kPfKeys * D * 2;          // one K or one V tile
  static constexpr int kPBytes = kPfTile * kPfKeys * 2;     // 128 rows x 128 B
  static constexpr int kBytes = kQBytes + 4 * kKVBytes + kPBytes + 256;  // the dynamic array is 1024-aligned
  static constexpr int kTmemCols = 256;                     // S: 64 columns, PV: D columns
};

__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// two float32 -> one register of two bf16 (round to nearest even), lo in the low half
__device__ __forceinline__ uint32_t pack_bf16x2_rn(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}

template <int D>
__global__ void __launch_bounds__(128, 2) attn_prefill_kernel(const __grid_constant__ CUtensorMap tmap_k,
                                                              const __grid_constant__ CUtensorMap tmap_v,
                                                              const PrefillParams p) {
  pdl_wait();  // nothing below may run ahead of the previous kernel in the stream
  using SM = PrefillSmem<D>;
  constexpr int kBoxes = D / 64;
  // CTAs start in the order of their linear index; under the causal mask the last query tile of a sequence has
  // the most key tiles to walk, so the index is unfolded heaviest tile first (all heads and sequences of the
  // last query tile, then the one before it, ...) and the short tiles fill the tail of the launch.
  const int lin = blockIdx.x + gridDim.x * (blockIdx.y + gridDim.y * blockIdx.z);
  const int hb = gridDim.y * gridDim.z;
  const int qb = (int)gridDim.x - 1 - lin / hb, h = (lin % hb) % (int)gridDim.y, b = (lin % hb) / (int)gridDim.y;
  const int hk = h / (p.Hq / p.Hkv);
  const int q0 = qb * kPfTile;                    // first query index of this CTA
  const int rows_valid = min(kPfTile, p.T - q0);
  // cross-attention: as if every query sat at the context's last position and the sequence began at -T
  const int kv_len = p.cross ? (int)max(1LL, min((long long)p.positions[b], p.max_len)) : 0;
  const int start = p.cross ? kv_len - p.T : p.positions[b];
  const int last_pos = p.cross ? kv_len - 1 : start + q0 + rows_valid - 1;  // highest key position any row may see
  const int win = p.window;
  // with a sliding window the tiles below the first row's window are never loaded
  const int j_lo = win >= 0 ? max(0, start + q0 - win) / kPfKeys : 0;
  const int n_tiles = last_pos / kPfKeys + 1 - j_lo;  // tiles j_lo .. j_lo + n_tiles - 1
  const int total_len = start + p.T;              // rows of the cache holding this sequence

  extern __shared__ __align__(1024) uint8_t smem[];  // swizzled tiles need 1024-byte alignment
  uint8_t* sQ = smem;
  uint8_t* sKV = sQ + SM::kQBytes;                // stage s: K at s*2*kKVBytes, V right after
  uint8_t* sP = sKV + 4 * SM::kKVBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sP + SM::kPBytes);
  uint64_t* bar_kv = bars;      // [2]
  uint64_t* bar_s = bars + 2;
  uint64_t* bar_o = bars + 3;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int tid = threadIdx.x, warp = tid >> 5;

  auto issue_tile = [&](int j) {  // thread 0 only
    const int s = j & 1;
    uint8_t* k_dst = sKV + s * 2 * SM::kKVBytes;
    uint8_t* v_dst = k_dst + SM::kKVBytes;
    mbar_arrive_expect_tx(bar_kv + s, 2 * SM::kKVBytes);
#pragma unroll
    for (int x = 0; x < kBoxes; ++x) {
      tma_load_4d(k_dst + x * SM::kKVHalfBytes, &tmap_k, bar_kv + s, x * 64, hk, (j_lo + j) * kPfKeys, b);
      tma_load_4d(v_dst + x * SM::kKVHalfBytes, &tmap_v, bar_kv + s, x * 64, hk, (j_lo + j) * kPfKeys, b);
    }
  };

  if (tid == 0) {
    mbar_init(bar_kv, 1);
    mbar_init(bar_kv + 1, 1);
    mbar_init(bar_s, 1);
    mbar_init(bar_o, 1);
    *abort_flag = 0;
    fence_mbar_init();
    issue_tile(0);
    if (n_tiles > 1) issue_tile(1);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, SM::kTmemCols);
    tmem_relinquish();
  }
  // Q rows -> shared memory (K-major, swizzled); rows past T are zero.
  {
    constexpr int kChunksPerRow = D / 8;
    for (int i = tid; i < kPfTile * kChunksPerRow; i += 128) {
      const int r = i / kChunksPerRow, c = i % kChunksPerRow;
      uint4 v = make_uint4(0, 0, 0, 0);
      if (r < rows_valid)
        v = __ldg(reinterpret_cast<const uint4*>(p.q + (((long long)b * p.T + q0 + r) * p.Hq + h) * D) + c);
      *reinterpret_cast<uint4*>(sQ + (c / 8) * SM::kHalfBytes + sw128_offset(r, c % 8)) = v;
    }
  }
  fence_proxy_async_smem();
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  pdl_trigger();  // tensor memory is allocated: the next kernel may be scheduled
  const uint32_t tmem_s = tmem_base;          // columns [0, 64)
  const uint32_t tmem_pv = tmem_base + 64;    // columns [64, 64 + D)
  const uint32_t lane_off = uint32_t(warp * 32) << 16;

  // Thread r owns query row r.  The output accumulates in tensor memory: the second MMA adds P V to it,
  // so the threads read it only once, at the end.  The scores of a tile are read from tensor memory once
  // (64 registers).  Exponentials are taken against a reference maximum m_ref that follows the running
  // maximum lazily: only when a tile's maximum exceeds it by more than kSlack (in the base-2 domain) is the
  // accumulator row -- and the running denominator -- rescaled; until then probabilities may be as
  // large as 2^kSlack, which bf16 and the float32 accumulator hold without loss of accuracy.  A row
  // that has seen no visible key yet keeps m_ref = -inf and contributes nothing.
  constexpr float kSlack = 8.0f;
  float m_ref = -INFINITY, l_run = 0.0f;
  const int qpos = p.cross ? kv_len - 1 : start + q0 + min(tid, rows_valid - 1);  // rows past T mirror the last valid row
  const float scale_log2 = p.sm_scale * 1.4426950408889634f;
  const int lo_vis = win >= 0 ? qpos - win : 0;  // lowest key position this row sees

  auto issue_qk = [&](int j) {  // thread 0: S = Q K_j^T into tensor memory, completion on bar_s
    const uint8_t* sK = sKV + (j & 1) * 2 * SM::kKVBytes;
    tc_fence_after_sync();
    constexpr uint32_t idesc = umma_idesc(kFmtBF16, kFmtBF16, 0, 0, 128, kPfKeys);
#pragma unroll
    for (int k = 0; k < D / 16; ++k) {
      const uint32_t box = k / 4, off = (k % 4) * 32;
      umma_f16(tmem_s, umma_desc_kmajor_sw128(smem_u32(sQ + box * SM::kHalfBytes) + off),
               umma_desc_kmajor_sw128(smem_u32(sK + box * SM::kKVHalfBytes) + off), idesc, k != 0);
    }
    umma_commit(bar_s);
  };

  bool ok = true;
  if (tid == 0) {
    ok = mbar_wait(bar_kv, 0, abort_flag, p.d_status, XAXB_DEVICE_TIMEOUT * 1000 + kSitePfKV);
    if (ok) issue_qk(0);
  }
  for (int j = 0; j < n_tiles; ++j) {
    const int s = j & 1;
    uint8_t* sV = sKV + s * 2 * SM::kKVBytes + SM::kKVBytes;
    const int kv0 = (j_lo + j) * kPfKeys;
    // ---- scores of tile j: one read from tensor memory ------------------------------------------
    ok = ok && mbar_wait(bar_s, j & 1, abort_flag, p.d_status, XAXB_DEVICE_TIMEOUT * 1000 + kSitePfS);
    uint32_t sreg[kPfKeys];
    __syncwarp();  // the tensor-memory loads below are warp-wide
    if (ok) {
      tc_fence_after_sync();
#pragma unroll
      for (int c0 = 0; c0 < kPfKeys; c0 += 32) {
        uint32_t r[32];
        tmem_ld_x32(tmem_s + lane_off + c0, r);
#pragma unroll
        for (int i = 0; i < 32; ++i) sreg[c0 + i] = r[i];
      }
      tmem_ld_wait();
    }
    // some (row, col) of this tile is masked: above the diagonal (past the context's end for
    // cross-attention), or below some row's window
    const bool diag = kv0 + kPfKeys - 1 > (p.cross ? kv_len - 1 : start + q0) || (win >= 0 && kv0 < last_pos - win);
    // column i of the tile is visible to this row iff lim_lo <= i <= lim_hi
    const int lim_hi = qpos - kv0, lim_lo = lo_vis - kv0;
    float m_tile = -INFINITY;
    if (diag) {
#pragma unroll
      for (int i = 0; i < kPfKeys; ++i)
        if (i <= lim_hi && i >= lim_lo) m_tile = fmaxf(m_tile, __uint_as_float(sreg[i]));
    } else {
#pragma unroll
      for (int i = 0; i < kPfKeys; ++i) m_tile = fmaxf(m_tile, __uint_as_float(sreg[i]));
    }
    m_tile *= scale_log2;
    // ---- the previous tile's P V must be complete before its operands (sP, the V stage) or the
    // accumulator are touched; its K/V stage is then free for tile j + 1's successor
    if (j > 0) {
      ok = ok && mbar_wait(bar_o, (j - 1) & 1, abort_flag, p.d_status, XAXB_DEVICE_TIMEOUT * 1000 + kSitePfO);
      if (ok) tc_fence_after_sync();
      if (tid == 0 && ok && j + 1 < n_tiles) issue_tile(j + 1);  // into the stage tile j - 1 used
    }
    // ---- lazy rescale of the row's accumulator --------------------------------------------------
    const bool grow = m_tile > m_ref + kSlack;  // (false while both are -inf)
    const bool first = m_ref == -INFINITY && m_tile > -INFINITY;
    __syncwarp();
    if (__any_sync(0xffffffffu, ok && grow && !first && j > 0)) {
      const float alpha = (grow && !first) ? exp2f(m_ref - m_tile) : 1.0f;
#pragma unroll 1
      for (int c0 = 0; c0 < D; c0 += 32) {
        uint32_t r[32];
        tmem_ld_x32(tmem_pv + lane_off + c0, r);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
        tmem_st_x32(tmem_pv + lane_off + c0, r);
      }
      tmem_st_wait();
      l_run *= alpha;
    }
    if (grow || first) m_ref = m_tile;
    // ---- probabilities -> shared memory (bf16, the A operand of the second MMA) -------------------
    // One multiply-add and one ex2.approx per score (arguments are <= kSlack: no range handling needed;
    // -inf and very negative arguments give 0), one cvt per pair.  Tiles that the diagonal or the sequence
    // end crosses take the branch with the per-column tests, the others (most of a long sequence) skip them.
    const float m_use = m_ref == -INFINITY ? 0.0f : m_ref;
    float l_tile = 0.0f;
    if (diag) {
#pragma unroll
      for (int c0 = 0; c0 < kPfKeys; c0 += 8) {
        uint32_t packed[4];
#pragma unroll
        for (int i = 0; i < 8; i += 2) {
          float e0 = ex2_approx(fmaf(__uint_as_float(sreg[c0 + i]), scale_log2, -m_use));
          float e1 = ex2_approx(fmaf(__uint_as_float(sreg[c0 + i + 1]), scale_log2, -m_use));
          if (c0 + i > lim_hi || c0 + i < lim_lo) e0 = 0.0f;
          if (c0 + i + 1 > lim_hi || c0 + i + 1 < lim_lo) e1 = 0.0f;
          l_tile += e0 + e1;
          packed[i / 2] = pack_bf16x2_rn(e0, e1);
        }
        *reinterpret_cast<uint4*>(sP + sw128_offset(tid, c0 / 8)) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
      }
    } else {
#pragma unroll
      for (int c0 = 0; c0 < kPfKeys; c0 += 8) {
        uint32_t packed[4];
#pragma unroll
        for (int i = 0; i < 8; i += 2) {
          const float e0 = ex2_approx(fmaf(__uint_as_float(sreg[c0 + i]), scale_log2, -m_use));
          const float e1 = ex2_approx(fmaf(__uint_as_float(sreg[c0 + i + 1]), scale_log2, -m_use));
          l_tile += e0 + e1;
          packed[i / 2] = pack_bf16x2_rn(e0, e1);
        }
        *reinterpret_cast<uint4*>(sP + sw128_offset(tid, c0 / 8)) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
      }
    }
    l_run += l_tile;
    // rows of the tile past the sequence's last cached token may hold anything; the mask zeroed
    // their probabilities, and V is cleared so that 0 * garbage stays 0
    ok = ok && mbar_wait(bar_kv + s, (j >> 1) & 1, abort_flag, p.d_status, XAXB_DEVICE_TIMEOUT * 1000 + kSitePfKV);
    if (ok && tid < kPfKeys && kv0 + tid >= total_len) {
#pragma unroll
      for (int c = 0; c < D / 8; ++c)
        *reinterpret_cast<uint4*>(sV + (c / 8) * SM::kKVHalfBytes + sw128_offset(tid, c % 8)) = make_uint4(0, 0, 0, 0);
    }
    fence_proxy_async_smem();
    tc_fence_before_sync();
    ok = __syncthreads_and(ok);
    if (!ok) break;
    // ---- O += P V; then, behind it in the tensor pipe, the next tile's scores --------------------
    if (tid == 0) {
      tc_fence_after_sync();
      constexpr uint32_t idesc = umma_idesc(kFmtBF16, kFmtBF16, 0, 1, 128, D);
#pragma unroll
      for (int k = 0; k < kPfKeys / 16; ++k) {
        umma_f16(tmem_pv, umma_desc_kmajor_sw128(smem_u32(sP) + k * 32),
                 umma_desc_mnmajor_sw128(smem_u32(sV) + k * 16 * 128, SM::kKVHalfBytes), idesc, (j | k) != 0);
      }
      umma_commit(bar_o);
      if (j + 1 < n_tiles) {
        if (mbar_wait(bar_kv + ((j + 1) & 1), ((j + 1) >> 1) & 1, abort_flag, p.d_status,
                      XAXB_DEVICE_TIMEOUT * 1000 + kSitePfKV))
          issue_qk(j + 1);
      }
    }
  }
  if (ok) {
    ok = mbar_wait(bar_o, (n_tiles - 1) & 1, abort_flag, p.d_status, XAXB_DEVICE_TIMEOUT * 1000 + kSitePfO);
    if (ok) tc_fence_after_sync();
  }

  __syncwarp();
  if (ok) {
    const float inv = 1.0f / l_run;
    __nv_bfloat16* dst = p.out + (((long long)b * p.T + q0 + tid) * p.Hq + h) * D;
#pragma unroll 1
    for (int c0 = 0; c0 < D; c0 += 32) {
      uint32_t r[32];
      tmem_ld_x32(tmem_pv + lane_off + c0, r);  // (warp-wide: rows past T read their lanes too)
      tmem_ld_wait();
      if (tid < rows_valid) {
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint4 v;
          uint32_t* w = reinterpret_cast<uint32_t*>(&v);
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const uint32_t lo = __bfloat16_as_ushort(__float2bfloat16_rn(__uint_as_float(r[c * 8 + 2 * i]) * inv));
            const uint32_t hi = __bfloat16_as_ushort(__float2bfloat16_rn(__uint_as_float(r[c * 8 + 2 * i + 1]) * inv));
            w[i] = lo | (hi << 16);
          }
          *reinterpret_cast<uint4*>(dst + c0 + c * 8) = v;
        }
      }
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, SM::kTmemCols);
  }
}

static int make_cache_tmap_pf(const Ctx* ctx, CUtensorMap* map, const void* cache, int64_t B, int64_t max_len,
                              int64_t Hkv, int64_t D) {
  const uint64_t dims[4] = {(uint64_t)D, (uint64_t)Hkv, (uint64_t)max_len, (uint64_t)B};
  const uint64_t strides[3] = {(uint64_t)D * 2, (uint64_t)Hkv * D * 2, (uint64_t)max_len * Hkv * D * 2};
  const uint32_t box[4] = {64, 1, (uint32_t)kPfKeys, 1};
  return make_tmap_4d(ctx, map, cache, 2, dims, strides, box);
}

}  // namespace xaxb

using namespace xaxb;

static int prefill_launch(xaxb_ctx* ctx_, void* stream, const void* q_rot_bf16, const void* k_cache_bf16,
                          const void* v_cache_bf16, const int32_t* positions, int64_t B, int64_t T, int64_t Hq,
                          int64_t Hkv, int64_t D, int64_t max_len, float softmax_scale, int64_t window, void* out_bf16,
                          int cross = 0) {
  if (!ctx_ || !q_rot_bf16 || !k_cache_bf16 || !v_cache_bf16 || !positions || !out_bf16 || B <= 0 || T <= 0 ||
      Hq <= 0 || Hkv <= 0 || max_len <= 0) {
    set_last_error("attn_prefill: null pointer or non-positive shape");
    return XAXB_BAD_ARGUMENT;
  }
  if (Hq % Hkv != 0 || (D != 128 && D != 64) || Hq > 65535 || B > 65535) {
    set_last_error("attn_prefill: needs head_dim 64 or 128 and Hq a multiple of Hkv");
    return XAXB_UNSUPPORTED;
  }
  if ((reinterpret_cast<uintptr_t>(q_rot_bf16) | reinterpret_cast<uintptr_t>(out_bf16)) & 15) return XAXB_BAD_ARGUMENT;
  const Ctx* ctx = reinterpret_cast<const Ctx*>(ctx_);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  CUtensorMap tk, tv;
  int rc = make_cache_tmap_pf(ctx, &tk, k_cache_bf16, B, max_len, Hkv, D);
  if (rc) return rc;
  rc = make_cache_tmap_pf(ctx, &tv, v_cache_bf16, B, max_len, Hkv, D);
  if (rc) return rc;
  PrefillParams p;
  p.q = static_cast<const __nv_bfloat16*>(q_rot_bf16);
  p.out = static_cast<__nv_bfloat16*>(out_bf16);
  p.positions = positions;
  p.T = (int)T, p.Hq = (int)Hq, p.Hkv = (int)Hkv;
  p.sm_scale = softmax_scale;
  p.window = window < 0 ? -1 : (window > 0x3fffffff ? 0x3fffffff : (int)window);
  p.cross = cross;
  p.max_len = max_len;
  p.d_status = ctx->d_status;
  dim3 grid((unsigned)((T + kPfTile - 1) / kPfTile), (unsigned)Hq, (unsigned)B);
  if (D == 128) {
    if (int rc2 = ensure_dynamic_smem<attn_prefill_kernel<128>>(ctx, PrefillSmem<128>::kBytes, "attn_prefill_kernel"))
      return rc2;
    launch_kernel(attn_prefill_kernel<128>, grid, dim3(128), PrefillSmem<128>::kBytes, s, 1, tk, tv, p);
  } else {
    if (int rc2 = ensure_dynamic_smem<attn_prefill_kernel<64>>(ctx, PrefillSmem<64>::kBytes, "attn_prefill_kernel"))
      return rc2;
    launch_kernel(attn_prefill_kernel<64>, grid, dim3(128), PrefillSmem<64>::kBytes, s, 1, tk, tv, p);
  }
  return check_launch("attn_prefill_kernel");
}

extern "C" int xaxb_attn_prefill(xaxb_ctx* ctx_, void* stream, const void* q_rot_bf16, const void* k_cache_bf16,
                                 const void* v_cache_bf16, const int32_t* positions, int64_t B, int64_t T, int64_t Hq,
                                 int64_t Hkv, int64_t D, int64_t max_len, float softmax_scale, void* out_bf16) {
  return prefill_launch(ctx_, stream, q_rot_bf16, k_cache_bf16, v_cache_bf16, positions, B, T, Hq, Hkv, D, max_len,
                        softmax_scale, -1, out_bf16);
}

extern "C" int xaxb_attn_prefill_window(xaxb_ctx* ctx_, void* stream, const void* q_rot_bf16, const void* k_cache_bf16,
                                        const void* v_cache_bf16, const int32_t* positions, int64_t B, int64_t T,
                                        int64_t Hq, int64_t Hkv, int64_t D, int64_t max_len, float softmax_scale,
                                        int64_t window, void* out_bf16) {
  return prefill_launch(ctx_, stream, q_rot_bf16, k_cache_bf16, v_cache_bf16, positions, B, T, Hq, Hkv, D, max_len,
                        softmax_scale, window, out_bf16);
}

extern "C" int xaxb_attn_cross(xaxb_ctx* ctx_, void* stream, const void* q_bf16, const void* k_bf16, const void* v_bf16,
                               const int32_t* kv_lens, int64_t B, int64_t T, int64_t Hq, int64_t Hkv, int64_t D,
                               int64_t max_len, float softmax_scale, void* out_bf16) {
  return prefill_launch(ctx_, stream, q_bf16, k_bf16, v_bf16, kv_lens, B, T, Hq, Hkv, D, max_len, softmax_scale, -1,
                        out_bf16, 1);
}
