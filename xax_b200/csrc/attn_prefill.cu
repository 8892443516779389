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
  int q_tiles;  // query tiles per (sequence, head)
  int n_items;  // q_tiles * Hq * B work items
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
  static constexpr int kTmemCols = 256;                     // S: two buffers of 64 columns, PV: D columns
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

constexpr int kPfThreads = 192;  // warps 0-3: one query row per thread; warp 4: MMA issue; warp 5: TMA loads

// Roles.  Issuing an MMA or a TMA instruction, or finding an mbarrier complete, costs the issuing thread about
// a hundred cycles each, and a tile needs twelve MMAs, four loads and half a dozen waits: 1500 of the 3050
// cycles a tile took when one of the softmax threads also did the issuing and the other 127 waited for it.
// So one lane of warp 4 issues the MMAs, one lane of warp 5 the loads, and the scores are double buffered in
// tensor memory: while the softmax warps work on tile j, Q K_{j+1}^T is already queued, and the softmax warps
// go from one tile to the next without waiting for the tensor pipe.
//
// Barriers (all in shared memory of this CTA):
//   bar_k[2], bar_v[2]   a K / V tile has landed (TMA transaction bytes); tile j uses slot j & 1
//   bar_s[2]             S buffer j & 1 holds Q K_j^T (MMA commit); also: K slot j & 1 may be reloaded
//   bar_p                the probabilities of tile j are in shared memory, fenced (4 arrivals); also: the
//                        softmax warps have read S buffer j & 1 out of tensor memory
//   bar_o                P_j V_j has been added to the accumulator (MMA commit); also: V slot j & 1 and the
//                        P buffer may be rewritten
// (j counts the key tiles a CTA has walked since it started, over all its work items.)
//
// Work distribution.  A work item is one 128-query tile of one head of one sequence.  Under the causal mask
// the items of a sequence differ eightfold and more in their number of key tiles, and an SM that holds two
// CTAs was seen to take a new CTA only once both had left (41 us for the config-2 launch where the work is
// 27 us per slot).  So the launch is one resident wave of at most two CTAs per SM, and CTA c of G walks items
// c, 2G-1-c, 2G+c, ... of the list ordered heaviest first (boustrophedon: the CTA that drew the heaviest item
// of one round draws the lightest of the next), which levels the key tiles per CTA to within one item.
template <int D>
__global__ void __launch_bounds__(kPfThreads, 2) attn_prefill_kernel(const __grid_constant__ CUtensorMap tmap_k,
                                                                     const __grid_constant__ CUtensorMap tmap_v,
                                                                     const PrefillParams p) {
  pdl_wait();  // nothing below may run ahead of the previous kernel in the stream
  using SM = PrefillSmem<D>;
  constexpr int kBoxes = D / 64;
  const int win = p.window;

  extern __shared__ __align__(1024) uint8_t smem[];  // swizzled tiles need 1024-byte alignment
  uint8_t* sQ = smem;
  uint8_t* sK = sQ + SM::kQBytes;                 // two K tiles
  uint8_t* sV = sK + 2 * SM::kKVBytes;            // two V tiles
  uint8_t* sP = sV + 2 * SM::kKVBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sP + SM::kPBytes);
  uint64_t* bar_k = bars;          // [2]
  uint64_t* bar_v = bars + 2;      // [2]
  uint64_t* bar_s = bars + 4;      // [2]
  uint64_t* bar_p = bars + 6;
  uint64_t* bar_o = bars + 7;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

  if (tid == 0) {
    for (int i = 0; i < 6; ++i) mbar_init(bars + i, 1);
    mbar_init(bar_p, 4);
    mbar_init(bar_o, 1);
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, SM::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  pdl_trigger();  // tensor memory is allocated: the next kernel may be scheduled
  const uint32_t tmem_s = tmem_base;                      // S buffers: columns [0, 64) and [64, 128)
  const uint32_t tmem_pv = tmem_base + 2 * kPfKeys;       // columns [128, 128 + D)

  const int G = gridDim.x, cta = blockIdx.x;
  const int hb = p.Hq * (p.n_items / (p.q_tiles * p.Hq));  // heads x sequences
  int gb = 0;  // key tiles walked by this CTA before the current item: barrier slots and parities follow gb + j
  for (int round = 0; round * G < p.n_items; ++round) {
    const int lin = round * G + ((round & 1) ? G - 1 - cta : cta);
    if (lin >= p.n_items) continue;  // (uniform over the CTA)
    // the list is ordered heaviest first: all heads and sequences of the last query tile, then the one before it, ...
    const int qb = p.q_tiles - 1 - lin / hb, h = (lin % hb) % p.Hq, b = (lin % hb) / p.Hq;
    const int hk = h / (p.Hq / p.Hkv);
    const int q0 = qb * kPfTile;                    // first query index of this item
    const int rows_valid = min(kPfTile, p.T - q0);
    // cross-attention: as if every query sat at the context's last position and the sequence began at -T
    const int kv_len = p.cross ? (int)max(1LL, min((long long)p.positions[b], p.max_len)) : 0;
    const int start = p.cross ? kv_len - p.T : p.positions[b];
    const int last_pos = p.cross ? kv_len - 1 : start + q0 + rows_valid - 1;  // highest key position any row may see
    // with a sliding window the tiles below the first row's window are never loaded
    const int j_lo = win >= 0 ? max(0, start + q0 - win) / kPfKeys : 0;
    const int n_tiles = last_pos / kPfKeys + 1 - j_lo;  // tiles j_lo .. j_lo + n_tiles - 1
    const int total_len = start + p.T;              // rows of the cache holding this sequence

    auto load_k = [&](int j) {  // loader only
      const int s = (gb + j) & 1;
      mbar_arrive_expect_tx(bar_k + s, SM::kKVBytes);
#pragma unroll
      for (int x = 0; x < kBoxes; ++x)
        tma_load_4d(sK + s * SM::kKVBytes + x * SM::kKVHalfBytes, &tmap_k, bar_k + s, x * 64, hk, (j_lo + j) * kPfKeys, b);
    };
    auto load_v = [&](int j) {  // loader only
      const int s = (gb + j) & 1;
      mbar_arrive_expect_tx(bar_v + s, SM::kKVBytes);
#pragma unroll
      for (int x = 0; x < kBoxes; ++x)
        tma_load_4d(sV + s * SM::kKVBytes + x * SM::kKVHalfBytes, &tmap_v, bar_v + s, x * 64, hk, (j_lo + j) * kPfKeys, b);
    };

    // The previous item's MMAs are complete (its softmax warps waited for the last of them before the barrier
    // that ended the item), so every shared-memory tile is free: the first K / V tiles are requested before the
    // query tile is staged, and land while it is.
    if (warp == 5 && lane == 0) {
      load_k(0);
      load_v(0);
      if (n_tiles > 1) {
        load_k(1);
        load_v(1);
      }
    }
    // Q rows -> shared memory (K-major, swizzled); rows past T are zero.  All of a thread's loads are issued
    // before the first store so that they overlap.
    {
      constexpr int kChunksPerRow = D / 8;
      constexpr int kPerThread = (kPfTile * kChunksPerRow + kPfThreads - 1) / kPfThreads;
      uint4 qv[kPerThread];
#pragma unroll
      for (int u = 0; u < kPerThread; ++u) {
        const int i = tid + u * kPfThreads;
        const int r = i / kChunksPerRow, c = i % kChunksPerRow;
        qv[u] = make_uint4(0, 0, 0, 0);
        if (i < kPfTile * kChunksPerRow && r < rows_valid)
          qv[u] = __ldg(reinterpret_cast<const uint4*>(p.q + (((long long)b * p.T + q0 + r) * p.Hq + h) * D) + c);
      }
#pragma unroll
      for (int u = 0; u < kPerThread; ++u) {
        const int i = tid + u * kPfThreads;
        const int r = i / kChunksPerRow, c = i % kChunksPerRow;
        if (i < kPfTile * kChunksPerRow)
          *reinterpret_cast<uint4*>(sQ + (c / 8) * SM::kHalfBytes + sw128_offset(r, c % 8)) = qv[u];
      }
    }
    fence_proxy_async_smem();
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    bool ok = true;

  if (warp == 5) {
    // ------------------------------------------------------------------ loader (one lane)
    if (lane == 0) {  // (tiles 0 and 1 were requested before the query tile was staged)
      for (int j = 0; j < n_tiles && ok; ++j) {
        const int g = gb + j;
        // the V slot of tile j + 1 was last read by P V of tile j - 1
        if (j >= 1 && j + 1 < n_tiles) {
          ok = mbar_wait(bar_o, (g - 1) & 1, abort_flag, p.d_status, XAXB_DEVICE_TIMEOUT * 1000 + kSitePfO);
          if (!ok) break;
          load_v(j + 1);
        }
        // the K slot of tile j + 2 is tile j's, free once Q K_j^T has run
        if (j + 2 < n_tiles) {
          ok = mbar_wait(bar_s + (g & 1), (g >> 1) & 1, abort_flag, p.d_status, XAXB_DEVICE_TIMEOUT * 1000 + kSitePfS);
          if (!ok) break;
          load_k(j + 2);
        }
      }
    }
  } else if (warp == 4) {
    // ------------------------------------------------------------------ MMA issuer (one lane)
    if (lane == 0) {
      auto issue_qk = [&](int j) {  // S buffer j & 1 = Q K_j^T, completion on bar_s[j & 1]
        const int s = (gb + j) & 1;
        const uint8_t* k_src = sK + s * SM::kKVBytes;
        tc_fence_after_sync();
        constexpr uint32_t idesc = umma_idesc(kFmtBF16, kFmtBF16, 0, 0, 128, kPfKeys);
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t box = k / 4, off = (k % 4) * 32;
          umma_f16(tmem_s + s * kPfKeys, umma_desc_kmajor_sw128(smem_u32(sQ + box * SM::kHalfBytes) + off),
                   umma_desc_kmajor_sw128(smem_u32(k_src + box * SM::kKVHalfBytes) + off), idesc, k != 0);
        }
        umma_commit(bar_s + s);
      };
      ok = mbar_wait(bar_k + (gb & 1), (gb >> 1) & 1, abort_flag, p.d_status, XAXB_DEVICE_TIMEOUT * 1000 + kSitePfKV);
      if (ok) issue_qk(0);
      for (int j = 0; j < n_tiles && ok; ++j) {
        const int g = gb + j;
        // The next tile's scores, queued while the softmax warps are busy with tile j.  Their S buffer was
        // tile j - 1's, which the softmax warps had read out before they signalled bar_p for tile j - 1
        // (waited for below, one iteration ago).
        if (j + 1 < n_tiles) {
          ok = mbar_wait(bar_k + ((g + 1) & 1), ((g + 1) >> 1) & 1, abort_flag, p.d_status,
                         XAXB_DEVICE_TIMEOUT * 1000 + kSitePfKV);
          if (!ok) break;
          issue_qk(j + 1);
        }
        // O += P_j V_j once the probabilities (and V_j) are in shared memory
        ok = mbar_wait(bar_p, g & 1, abort_flag, p.d_status, XAXB_DEVICE_TIMEOUT * 1000 + kSitePfO);
        ok = ok && mbar_wait(bar_v + (g & 1), (g >> 1) & 1, abort_flag, p.d_status, XAXB_DEVICE_TIMEOUT * 1000 + kSitePfKV);
        if (!ok) break;
        tc_fence_after_sync();
        const uint8_t* v_src = sV + (g & 1) * SM::kKVBytes;
        constexpr uint32_t idesc = umma_idesc(kFmtBF16, kFmtBF16, 0, 1, 128, D);
#pragma unroll
        for (int k = 0; k < kPfKeys / 16; ++k) {
          umma_f16(tmem_pv, umma_desc_kmajor_sw128(smem_u32(sP) + k * 32),
                   umma_desc_mnmajor_sw128(smem_u32(v_src) + k * 16 * 128, SM::kKVHalfBytes), idesc, (j | k) != 0);
        }
        umma_commit(bar_o);
      }
    }
  } else {
    // ------------------------------------------------------------------ softmax: thread r owns query row r
    // The output accumulates in tensor memory: the second MMA adds P V to it, so the threads read it only
    // once, at the end.  The scores of a tile are read from tensor memory once (64 registers).  Exponentials
    // are taken against a reference maximum m_ref that follows the running maximum lazily: only when a tile's
    // maximum exceeds it by more than kSlack (in the base-2 domain) is the accumulator row -- and the running
    // denominator -- rescaled; until then probabilities may be as large as 2^kSlack, which bf16 and the
    // float32 accumulator hold without loss of accuracy.  A row that has seen no visible key yet keeps
    // m_ref = -inf and contributes nothing.
    const uint32_t lane_off = uint32_t(warp * 32) << 16;
    constexpr float kSlack = 8.0f;
    float m_ref = -INFINITY, l_run = 0.0f;
    const int qpos = p.cross ? kv_len - 1 : start + q0 + min(tid, rows_valid - 1);  // rows past T mirror the last valid row
    const float scale_log2 = p.sm_scale * 1.4426950408889634f;
    const int lo_vis = win >= 0 ? qpos - win : 0;  // lowest key position this row sees
    for (int j = 0; j < n_tiles; ++j) {
      const int g = gb + j, s = g & 1;
      uint8_t* v_tile = sV + s * SM::kKVBytes;
      const int kv0 = (j_lo + j) * kPfKeys;
      // ---- scores of tile j: one read from tensor memory ----------------------------------------
      ok = ok && mbar_wait(bar_s + s, (g >> 1) & 1, abort_flag, p.d_status, XAXB_DEVICE_TIMEOUT * 1000 + kSitePfS);
      uint32_t sreg[kPfKeys];
      __syncwarp();  // the tensor-memory loads below are warp-wide
      if (ok) {
        tc_fence_after_sync();
#pragma unroll
        for (int c0 = 0; c0 < kPfKeys; c0 += 32) {
          uint32_t r[32];
          tmem_ld_x32(tmem_s + s * kPfKeys + lane_off + c0, r);
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
      // ---- how far the reference maximum moves (the accumulator itself is rescaled further down) -------
      const bool grow = m_tile > m_ref + kSlack;  // (false while both are -inf)
      const bool first = m_ref == -INFINITY && m_tile > -INFINITY;
      const float alpha = (grow && !first) ? exp2f(m_ref - m_tile) : 1.0f;
      if (grow || first) m_ref = m_tile;
      l_run *= alpha;
      // ---- probabilities (bf16, the A operand of the second MMA), kept in registers for now --------------
      // One multiply-add and one ex2.approx per score (arguments are <= kSlack: no range handling needed;
      // -inf and very negative arguments give 0), one cvt per pair.  Tiles that the diagonal or the sequence
      // end crosses take the branch with the per-column tests, the others (most of a long sequence) skip them.
      const float m_use = m_ref == -INFINITY ? 0.0f : m_ref;
      float l_tile = 0.0f;
      uint32_t packed[kPfKeys / 2];
      if (diag) {
#pragma unroll
        for (int i = 0; i < kPfKeys; i += 2) {
          float e0 = ex2_approx(fmaf(__uint_as_float(sreg[i]), scale_log2, -m_use));
          float e1 = ex2_approx(fmaf(__uint_as_float(sreg[i + 1]), scale_log2, -m_use));
          if (i > lim_hi || i < lim_lo) e0 = 0.0f;
          if (i + 1 > lim_hi || i + 1 < lim_lo) e1 = 0.0f;
          l_tile += e0 + e1;
          packed[i / 2] = pack_bf16x2_rn(e0, e1);
        }
      } else {
#pragma unroll
        for (int i = 0; i < kPfKeys; i += 2) {
          const float e0 = ex2_approx(fmaf(__uint_as_float(sreg[i]), scale_log2, -m_use));
          const float e1 = ex2_approx(fmaf(__uint_as_float(sreg[i + 1]), scale_log2, -m_use));
          l_tile += e0 + e1;
          packed[i / 2] = pack_bf16x2_rn(e0, e1);
        }
      }
      // ---- the previous tile's P V must be complete before its P operand or the accumulator are touched;
      // by now it usually is (the exponentials above ran under it)
      if (j > 0) {
        ok = ok && mbar_wait(bar_o, (g - 1) & 1, abort_flag, p.d_status, XAXB_DEVICE_TIMEOUT * 1000 + kSitePfO);
        if (ok) tc_fence_after_sync();
      }
      // ---- lazy rescale of the row's accumulator ------------------------------------------------
      __syncwarp();
      if (__any_sync(0xffffffffu, ok && grow && !first && j > 0)) {
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
      }
#pragma unroll
      for (int c = 0; c < kPfKeys / 8; ++c)
        *reinterpret_cast<uint4*>(sP + sw128_offset(tid, c)) =
            make_uint4(packed[4 * c], packed[4 * c + 1], packed[4 * c + 2], packed[4 * c + 3]);
      l_run += l_tile;
      // rows of the tile past the sequence's last cached token may hold anything; the mask zeroed
      // their probabilities, and V is cleared so that 0 * garbage stays 0
      if (kv0 + kPfKeys > total_len) {  // (uniform over the CTA)
        ok = ok && mbar_wait(bar_v + s, (g >> 1) & 1, abort_flag, p.d_status, XAXB_DEVICE_TIMEOUT * 1000 + kSitePfKV);
        if (ok && tid < kPfKeys && kv0 + tid >= total_len) {
#pragma unroll
          for (int c = 0; c < D / 8; ++c)
            *reinterpret_cast<uint4*>(v_tile + (c / 8) * SM::kKVHalfBytes + sw128_offset(tid, c % 8)) = make_uint4(0, 0, 0, 0);
        }
      }
      fence_proxy_async_smem();
      tc_fence_before_sync();
      __syncwarp();
      if (!__all_sync(0xffffffffu, ok)) break;
      if (lane == 0) mbar_arrive(bar_p);  // the issuer queues O += P V behind this
    }
    if (ok) {
      ok = mbar_wait(bar_o, (gb + n_tiles - 1) & 1, abort_flag, p.d_status, XAXB_DEVICE_TIMEOUT * 1000 + kSitePfO);
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
  }
    // the item is done: every MMA has completed (the softmax warps waited for the last one), every load was
    // consumed; the shared-memory tiles, the S buffers and the accumulator are free for the next item
    tc_fence_before_sync();
    if (__syncthreads_or(!ok)) break;
    tc_fence_after_sync();
    gb += n_tiles;
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
  const long long q_tiles = (T + kPfTile - 1) / kPfTile, n_items = q_tiles * Hq * B;
  if (n_items > 0x7fffffffLL) {
    set_last_error("attn_prefill: more than 2^31 query tiles");
    return XAXB_UNSUPPORTED;
  }
  p.q_tiles = (int)q_tiles;
  p.n_items = (int)n_items;
  // one resident wave: two CTAs per SM (tensor memory: 2 x 256 columns), each walking its share of the items
  const long long slots = 2LL * ctx->num_sms;
  dim3 grid((unsigned)(n_items < slots ? n_items : slots));
  if (D == 128) {
    if (int rc2 = ensure_dynamic_smem<attn_prefill_kernel<128>>(ctx, PrefillSmem<128>::kBytes, "attn_prefill_kernel"))
      return rc2;
    launch_kernel(attn_prefill_kernel<128>, grid, dim3(kPfThreads), PrefillSmem<128>::kBytes, s, 1, tk, tv, p);
  } else {
    if (int rc2 = ensure_dynamic_smem<attn_prefill_kernel<64>>(ctx, PrefillSmem<64>::kBytes, "attn_prefill_kernel"))
      return rc2;
    launch_kernel(attn_prefill_kernel<64>, grid, dim3(kPfThreads), PrefillSmem<64>::kBytes, s, 1, tk, tv, p);
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
