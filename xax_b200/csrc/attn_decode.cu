// Kernel 3a: GQA decode attention over a bf16 KV cache, split over 128-token chunks.
//
// HBM-bound: every K and V row is read exactly once.  The chunks of one (sequence, kv head) are
// dealt to a few CTAs; a CTA walks its chunks one at a time, requesting the next chunk's K tile
// as soon as the first MMA has consumed the current one and the next V tile as soon as the
// second MMA has, so that loads stay in flight under the softmax.  The chunk's K and V tiles ([128 tokens x D] bf16) are brought in by TMA
// into 128-byte-swizzled shared memory and consumed in place by tcgen05.mma -- the threads
// never touch K or V (unless K is stored un-rotated, see below):
//
//   S^T[token, g] = K[token, :] . Q[g, :]      UMMA M = 128 tokens, N = 16 (G query heads of
//                                              the group, zero padded), K = D; A = K tile
//                                              (K-major), B = Q (K-major)
//   P = exp(S * scale - max)                   thread t owns token t: tcgen05.ld gives it the
//                                              G scores of its token; max / sum over tokens
//                                              are warp-shuffle + shared-memory reductions
//   O^T[d, g] = sum_token V[token, d] P[token, g]   UMMA M = 128 (for D = 64 the upper 64 rows
//                                              read a zeroed pad), N = 16, K = 128 tokens;
//                                              A = V tile (MN-major: D contiguous), B = P^T
//                                              written to shared memory as bf16 (K-major)
//
// Each CTA merges its chunks in registers (running max / sum / O^T) and writes one partial
// result to the workspace; a second kernel merges the partial results of a sequence with the
// usual log-sum-exp weights and writes bf16 output.
//
// With k_is_rotated = 0 the cache holds K as projected and the rotation is applied on load:
// after the TMA lands, thread t rotates row t of the K tile in shared memory with row
// (chunk start + t) of the cos/sin table (bf16 arithmetic in the reference's order) before
// the first MMA.
#include "common.cuh"
#include "quant_device.cuh"
#include "tp_device.cuh"

namespace xaxb {

constexpr int kChunk = 128;   // tokens per CTA
constexpr int kNPad = 16;     // UMMA N: query heads of one group, zero padded
constexpr int kSiteDecK = 11, kSiteDecV = 12, kSiteDecS = 13, kSiteDecO = 14;

// Where the merged, cast row of a sequence goes (see merge_cast_row).
struct MergeOut {
  uint4* out;  // bf16 row, may be null
  uint2* q;
  float* scale;
  float* inv_scale;
};

constexpr int kSiteDecPos = 15;

// Tokens sequence b attends to: positions[b] + 1, which must lie in 1 .. max_len.  A position
// outside that range is recorded (XAXB_CACHE_OVERFLOW, site 15) and clamped, so the kernels
// never divide by an empty softmax and never count rows past the cache as keys.
__device__ __forceinline__ int decode_len(const int32_t* positions, int b, long long max_len, int* d_status) {
  const int L = positions[b] + 1;
  if (L >= 1 && L <= max_len) return L;
  if (threadIdx.x == 0) atomicCAS(d_status, 0, XAXB_CACHE_OVERFLOW * 1000 + kSiteDecPos);
  return L < 1 ? 1 : (int)max_len;
}

// Chunks a sequence of L cached tokens contributes when its last token looks back `window`
// positions (< 0: all of them).
__host__ __device__ __forceinline__ int decode_chunks(int L, int window) {
  const int n = (L + kChunk - 1) / kChunk;
  const int lo = window >= 0 ? (L - 1 - window > 0 ? L - 1 - window : 0) : 0;
  return n - lo / kChunk;
}

struct DecodeParams {
  const __nv_bfloat16* q;      // [B, Hq, D] rotated
  const int32_t* positions;    // [B]; attend to rows 0 .. positions[b]
  int Hq, Hkv, G;
  long long max_len;
  float sm_scale;
  int k_is_rotated;
  const __nv_bfloat16* cos_t;  // [table_len, D/2]
  const __nv_bfloat16* sin_t;
  long long table_len;
  float* ws_o;   // [B, Hq, max_chunks, D]
  float* ws_ml;  // [B, Hq, max_chunks, 2]
  int max_chunks;
  int window;  // sliding window: the query at position q sees keys q - window .. q; < 0 = unlimited
  int* d_status;
  // Fused append (qkv != nullptr): the step's new token has not been written to the cache yet.  Row b of
  // qkv -- the fused projection's output, [q heads | k heads | v heads] x D, row stride qkv_ld -- holds
  // its query, key and value.  Every CTA rotates the query heads of its group as it stages them; the one
  // CTA that owns the chunk of position positions[b] rotates the new key (unless K is stored
  // un-rotated), places key and value in the row of its K / V tiles in shared memory where the cache
  // row will be, and writes them to the cache.  This replaces the append kernel of a decode step.
  const __nv_bfloat16* qkv;
  long long qkv_ld;
  __nv_bfloat16* k_cache;  // [B, max_len, Hkv, D]
  __nv_bfloat16* v_cache;
};

template <int D>
struct DecodeSmem {
  static constexpr int kTileBytes = kChunk * D * 2;           // one K or V tile
  static constexpr int kHalfBytes = kChunk * 128;             // one 64-element-wide TMA box
  static constexpr int kQBytes = kNPad * D * 2;
  static constexpr int kPBytes = kNPad * kChunk * 2;
  static constexpr int kVBytes = 2 * kHalfBytes;               // D = 64: second half is a zero pad
  static constexpr int kBytes = kTileBytes + kVBytes + kQBytes + kPBytes + 1024 /*alignment*/ + 1024;
};

// Merge + per-token cast of one sequence's row [Hq * D] (what the output projection consumes):
// the partial results of ALL its query heads are combined with log-sum-exp weights, kept in
// registers, the row's amax is reduced and e4m3 bytes are written with the row's scale -- the
// same result as the merge kernel followed by the per-token cast, without the bf16 round trip.
// Work item = (head, 8 consecutive dims); Hq * D <= 4096, so at most 512 / NT items per thread.
// Called by all NT threads of a CTA.  kFresh: the partial results were written by other CTAs of
// a kernel that is still running, so they are read past the (non-coherent) L1.  (Merging inside
// the attention kernel -- the CTA that finishes a sequence last -- was tried: the fence and the
// ticket each CTA then needs before it can leave cost more SM residency than the merge launch.)
template <bool kFresh>
__device__ __forceinline__ float ws_ld(const float* p) {
  return kFresh ? __ldcg(p) : *p;
}
template <bool kFresh>
__device__ __forceinline__ float4 ws_ld4(const float* p) {
  return kFresh ? __ldcg(reinterpret_cast<const float4*>(p)) : *reinterpret_cast<const float4*>(p);
}

template <int NT, bool kFresh>
__device__ __forceinline__ void merge_cast_row(const float* __restrict__ ws_o, const float* __restrict__ ws_ml, int b,
                                               int n, int Hq, int D, int max_chunks, const MergeOut mo,
                                               const TpRowMax& tp, int* d_status, float* s_max, float* s_inv_den,
                                               uint32_t* s_tp) {
  constexpr int kPer = 512 / NT;
  // (max, sum) of every partial result of the sequence, fetched by all threads at once: the
  // arithmetic below then runs from shared memory in the same order as before, without a chain of
  // dependent trips to L2 per head.  Up to kMlCache partial results per head are cached.
  constexpr int kMlCache = 16;
  __shared__ float s_ml[64 * kMlCache * 2];
  const bool cached = n <= kMlCache;
  if (cached) {
    for (int i = threadIdx.x; i < Hq * n; i += NT) {
      const int h = i / n, c = i - h * n;
      const long long base = ((long long)b * Hq + h) * max_chunks + c;
      const float2 v = kFresh ? __ldcg(reinterpret_cast<const float2*>(ws_ml + base * 2))
                              : *reinterpret_cast<const float2*>(ws_ml + base * 2);
      s_ml[(h * kMlCache + c) * 2] = v.x;
      s_ml[(h * kMlCache + c) * 2 + 1] = v.y;
    }
    __syncthreads();
  }
  for (int h = threadIdx.x; h < Hq; h += NT) {
    const long long base = ((long long)b * Hq + h) * max_chunks;
    float m = -INFINITY;
    float den = 0.0f;
    if (cached) {
      const float* ml = s_ml + h * kMlCache * 2;
      for (int c = 0; c < n; ++c) m = fmaxf(m, ml[c * 2]);
      for (int c = 0; c < n; ++c) den = fmaf(__expf(ml[c * 2] - m), ml[c * 2 + 1], den);
    } else {
      for (int c = 0; c < n; ++c) m = fmaxf(m, ws_ld<kFresh>(ws_ml + (base + c) * 2));
      for (int c = 0; c < n; ++c)
        den = fmaf(__expf(ws_ld<kFresh>(ws_ml + (base + c) * 2) - m), ws_ld<kFresh>(ws_ml + (base + c) * 2 + 1), den);
    }
    s_max[h] = m;
    s_inv_den[h] = 1.0f / den;
  }
  __syncthreads();
  const int dv = D / 8;
  const int items = Hq * dv;
  float v[kPer][8];
  uint32_t mbits = 0;
#pragma unroll
  for (int k = 0; k < kPer; ++k) {
    const int it = threadIdx.x + k * NT;
    if (it < items) {
      const int h = it / dv, d0 = (it % dv) * 8;
      const long long base = ((long long)b * Hq + h) * max_chunks;
      float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#pragma unroll 4
      for (int c = 0; c < n; ++c) {
        const float mc = cached ? s_ml[(h * kMlCache + c) * 2] : ws_ld<kFresh>(ws_ml + (base + c) * 2);
        const float w = __expf(mc - s_max[h]);
        const float4 lo = ws_ld4<kFresh>(ws_o + (base + c) * D + d0);
        const float4 hi = ws_ld4<kFresh>(ws_o + (base + c) * D + d0 + 4);
        acc[0] = fmaf(w, lo.x, acc[0]), acc[1] = fmaf(w, lo.y, acc[1]), acc[2] = fmaf(w, lo.z, acc[2]);
        acc[3] = fmaf(w, lo.w, acc[3]), acc[4] = fmaf(w, hi.x, acc[4]), acc[5] = fmaf(w, hi.y, acc[5]);
        acc[6] = fmaf(w, hi.z, acc[6]), acc[7] = fmaf(w, hi.w, acc[7]);
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        v[k][j] = bf16_round(acc[j] * s_inv_den[h]);
        mbits = max(mbits, mag_bits16(v[k][j]));
      }
      if (mo.out) mo.out[(long long)b * items + it] = pack8(v[k]);
    }
  }
  uint32_t row_bits = block_max_u32(mbits);
  // tensor-parallel runs: the other ranks hold the other heads of this token's row (the output
  // projection's input is split along its width); the scale comes from the amax over all of them
  if (tp.world > 1) row_bits = tp_cta_max_u32(tp, b, row_bits, s_tp, d_status, kSiteTpAttn);
  const float s = current_scale_from_amax(bf16_bits_to_float(row_bits));
#pragma unroll
  for (int k = 0; k < kPer; ++k) {
    const int it = threadIdx.x + k * NT;
    if (it < items) mo.q[(long long)b * items + it] = quantize8f(v[k], s);
  }
  if (threadIdx.x == 0) {
    mo.scale[b] = s;
    mo.inv_scale[b] = 1.0f / s;
  }
}

__device__ __forceinline__ float warp_max_f32(float v) {
  float r;
  asm volatile("redux.sync.max.f32 %0, %1, 0xffffffff;" : "=f"(r) : "f"(v));
  return r;
}

// Rotate-on-load.  A warp owns 32 rows of every K tile of its CTA and walks them a few rows at a time:
// D/16 neighbouring lanes share a row, lane l taking 16-byte piece l % (D/16) of the row's first half and
// the piece it pairs with in the second half, so that one warp-wide load of cos (or sin) values reads whole,
// consecutive table rows -- every byte the memory system moves is used; with a thread per row each load
// touched 32 different rows and half of every sector fetched was thrown away.  The table values
// are fetched into registers one tile ahead -- right after the previous tile was rotated -- so that they
// have arrived by the time the K tile lands; the rotation itself then only touches shared memory.
// It is packed bf16 arithmetic: every product and every sum rounds to bf16 on its own, which is exactly
// the reference's bf16 op sequence (xax/arch/attention.py:510-515), six instructions per two pairs.
// Pair (i, i + D/2) lives in 16-byte piece i/8 of box (i / 64) and piece (i + D/2)/8 of the row.
template <int D>
struct RopeRow {
  static constexpr int kPieces = D / 16;           // 16-byte pieces of a table row = lanes per K row
  static constexpr int kRowsPerStep = 32 / kPieces;
  static constexpr int kSteps = 32 / kRowsPerStep;  // (= kPieces)
  uint4 c[kSteps], s[kSteps];
  int rows;  // rows of the tile that have a token and a table row
};

template <int D>
__device__ __forceinline__ void load_rope_row(RopeRow<D>& r, const DecodeParams& p, int tok0, int valid) {
  using R = RopeRow<D>;
  constexpr int half = D / 2;
  const long long in_table = p.table_len - tok0;
  r.rows = (int)max(0LL, min((long long)valid, in_table));
  const int lane = threadIdx.x & 31, piece = lane % R::kPieces;
  const int row0 = (threadIdx.x & ~31) + lane / R::kPieces;
#pragma unroll
  for (int i = 0; i < R::kSteps; ++i) {
    const int row = row0 + i * R::kRowsPerStep;
    if (row < r.rows) {
      const long long pos = tok0 + row;
      r.c[i] = __ldg(reinterpret_cast<const uint4*>(p.cos_t + pos * half) + piece);
      r.s[i] = __ldg(reinterpret_cast<const uint4*>(p.sin_t + pos * half) + piece);
    }
  }
}

template <int D>
__device__ __forceinline__ void rotate_k_row(uint8_t* sK, const RopeRow<D>& r) {
  using SM = DecodeSmem<D>;
  using R = RopeRow<D>;
  const int lane = threadIdx.x & 31, piece = lane % R::kPieces, piece2 = piece + R::kPieces;
  const int row0 = (threadIdx.x & ~31) + lane / R::kPieces;
#pragma unroll
  for (int i = 0; i < R::kSteps; ++i) {
    const int row = row0 + i * R::kRowsPerStep;
    if (row >= r.rows) break;
    uint4* p1 = reinterpret_cast<uint4*>(sK + (piece / 8) * SM::kHalfBytes + sw128_offset(row, piece % 8));
    uint4* p2 = reinterpret_cast<uint4*>(sK + (piece2 / 8) * SM::kHalfBytes + sw128_offset(row, piece2 % 8));
    uint4 a = *p1, bb = *p2;
    __nv_bfloat162* aw = reinterpret_cast<__nv_bfloat162*>(&a);
    __nv_bfloat162* bw = reinterpret_cast<__nv_bfloat162*>(&bb);
    const __nv_bfloat162* cw = reinterpret_cast<const __nv_bfloat162*>(&r.c[i]);
    const __nv_bfloat162* sw = reinterpret_cast<const __nv_bfloat162*>(&r.s[i]);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const __nv_bfloat162 x1 = aw[j], x2 = bw[j];
      // the _rn forms are never contracted into a fused multiply-add
      aw[j] = __hsub2_rn(__hmul2_rn(x1, cw[j]), __hmul2_rn(x2, sw[j]));
      bw[j] = __hadd2_rn(__hmul2_rn(x2, cw[j]), __hmul2_rn(x1, sw[j]));
    }
    *p1 = a;
    *p2 = bb;
  }
}

// Fused append: the new token's key -> row r_new of the K tile in shared memory and row t_new of the
// cache.  Threads 0 .. D/16 - 1, one pair of 16-byte pieces each; the tile has landed.
template <int D>
__device__ __forceinline__ void place_new_key(uint8_t* sK, const DecodeParams& p, int b, int hk, int t_new, int r_new) {
  using SM = DecodeSmem<D>;
  constexpr int kPairs = D / 16;
  const int c = threadIdx.x;
  if (c >= kPairs) return;
  const uint4* src = reinterpret_cast<const uint4*>(p.qkv + (long long)b * p.qkv_ld + (long long)(p.Hq + hk) * D);
  uint4 a = __ldg(src + c), bb = __ldg(src + c + kPairs);
  if (p.k_is_rotated) {
    const uint4* cr = reinterpret_cast<const uint4*>(p.cos_t + (long long)t_new * (D / 2));
    const uint4* sr = reinterpret_cast<const uint4*>(p.sin_t + (long long)t_new * (D / 2));
    rope_rotate_pieces(a, bb, __ldg(cr + c), __ldg(sr + c), a, bb);
  }
  const int c2 = c + kPairs;
  *reinterpret_cast<uint4*>(sK + (c / 8) * SM::kHalfBytes + sw128_offset(r_new, c % 8)) = a;
  *reinterpret_cast<uint4*>(sK + (c2 / 8) * SM::kHalfBytes + sw128_offset(r_new, c2 % 8)) = bb;
  uint4* dst = reinterpret_cast<uint4*>(p.k_cache + (((long long)b * p.max_len + t_new) * p.Hkv + hk) * D);
  dst[c] = a;
  dst[c2] = bb;
}

// Same for the value (copied as it is).  Threads 0 .. D/8 - 1, one 16-byte piece each.
template <int D>
__device__ __forceinline__ void place_new_value(uint8_t* sV, const DecodeParams& p, int b, int hk, int t_new, int r_new) {
  using SM = DecodeSmem<D>;
  const int c = threadIdx.x;
  if (c >= D / 8) return;
  const uint4 v =
      __ldg(reinterpret_cast<const uint4*>(p.qkv + (long long)b * p.qkv_ld + (long long)(p.Hq + p.Hkv + hk) * D) + c);
  *reinterpret_cast<uint4*>(sV + (c / 8) * SM::kHalfBytes + sw128_offset(r_new, c % 8)) = v;
  reinterpret_cast<uint4*>(p.v_cache + (((long long)b * p.max_len + t_new) * p.Hkv + hk) * D)[c] = v;
}

// One K or V tile -> shared memory.  A chunk that the sequence fills only in part (its last one) is
// fetched in boxes of 32 token rows through the second tensor map, only as many as hold tokens: the
// rows behind them keep whatever the previous tile left, which the softmax masks (K) and the threads
// clear (V) as they do for any row past the sequence end.  Fetching the whole 128-row box regardless
// cost 3 % of the traffic at a context of ~2100 tokens (64 wasted rows per sequence on average).
constexpr int kPartRows = 32;
template <int D>
__device__ __forceinline__ void load_tile(uint8_t* dst, const CUtensorMap* whole, const CUtensorMap* part,
                                          uint64_t* bar, int hk, int tok0, int b, int rows) {
  using SM = DecodeSmem<D>;
  constexpr int kBoxes = D / 64;
  if (rows > kChunk - kPartRows) {
    mbar_arrive_expect_tx(bar, SM::kTileBytes);
#pragma unroll
    for (int x = 0; x < kBoxes; ++x) tma_load_4d(dst + x * SM::kHalfBytes, whole, bar, x * 64, hk, tok0, b);
  } else {
    const int n = (rows + kPartRows - 1) / kPartRows;
    mbar_arrive_expect_tx(bar, n * kPartRows * D * 2);
#pragma unroll
    for (int x = 0; x < kBoxes; ++x)
      for (int j = 0; j < n; ++j)
        tma_load_4d(dst + x * SM::kHalfBytes + j * kPartRows * 128, part, bar, x * 64, hk, tok0 + j * kPartRows, b);
  }
}

// GT = the group size rounded up to a power of two: only GT of the 16 UMMA columns are read back,
// reduced and written as P^T.  (Column n of either product depends on row n of its B operand
// only, so whatever the unused rows of Q and P^T hold never reaches a column that is read.)
template <int D, int GT, bool kRotate>
__global__ void __launch_bounds__(128, 3) attn_decode_kernel(const __grid_constant__ CUtensorMap tmap_k,
                                                          const __grid_constant__ CUtensorMap tmap_v,
                                                          const __grid_constant__ CUtensorMap tmap_k_part,
                                                          const __grid_constant__ CUtensorMap tmap_v_part,
                                                          const DecodeParams p) {
  pdl_wait();  // nothing below may run ahead of the previous kernel in the stream
  using SM = DecodeSmem<D>;
  constexpr int kBoxes = D / 64;  // 128-byte-wide boxes per row
  const int first = blockIdx.x, stride = gridDim.x, hk = blockIdx.y, b = blockIdx.z;
  const int L = decode_len(p.positions, b, p.max_len, p.d_status);
  const int n_chunks = (L + kChunk - 1) / kChunk;
  // with a sliding window the chunks below the first visible token are never loaded
  const int lo_tok = p.window >= 0 ? max(0, L - 1 - p.window) : 0;
  const int c_lo = lo_tok / kChunk;
  if (c_lo + first >= n_chunks) return;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sK = smem;
  uint8_t* sV = sK + SM::kTileBytes;
  uint8_t* sQ = sV + SM::kVBytes;             // [kBoxes][16 rows x 128 B], swizzled
  uint8_t* sP = sQ + SM::kQBytes;             // [2][16 rows x 128 B], swizzled (128 tokens)
  uint64_t* bars = reinterpret_cast<uint64_t*>(sP + SM::kPBytes);
  uint64_t* bar_k = bars;
  uint64_t* bar_v = bars + 1;
  uint64_t* bar_s = bars + 2;
  uint64_t* bar_o = bars + 3;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  float* red_max = reinterpret_cast<float*>(tmem_slot + 2);  // [4 warps][16]
  float* red_sum = red_max + 4 * kNPad;                       // [4 warps][16]

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

  if (tid == 0) {
    mbar_init(bar_k, 1);
    mbar_init(bar_v, 1);
    mbar_init(bar_s, 1);
    mbar_init(bar_o, 1);
    *abort_flag = 0;
    fence_mbar_init();
    const int t0 = (c_lo + first) * kChunk;
    load_tile<D>(sK, &tmap_k, &tmap_k_part, bar_k, hk, t0, b, min(kChunk, L - t0));
    load_tile<D>(sV, &tmap_v, &tmap_v_part, bar_v, hk, t0, b, min(kChunk, L - t0));
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 32);
    tmem_relinquish();
  }

  const bool append = p.qkv != nullptr;
  const int t_new = L - 1, c_new = t_new / kChunk, r_new = t_new % kChunk;  // the step's new token
  // Q of this group -> shared memory, K-major rows of D elements; rows G .. GT-1 zero.
  if (append) {  // ... rotated here, from the fused projection's output
    constexpr int kPairs = D / 16;
    const uint4* cr = reinterpret_cast<const uint4*>(p.cos_t + (long long)t_new * (D / 2));
    const uint4* sr = reinterpret_cast<const uint4*>(p.sin_t + (long long)t_new * (D / 2));
    for (int i = tid; i < GT * kPairs; i += 128) {
      const int g = i / kPairs, c = i % kPairs, c2 = c + kPairs;
      uint4 o1 = make_uint4(0, 0, 0, 0), o2 = o1;
      if (g < p.G) {
        const uint4* src =
            reinterpret_cast<const uint4*>(p.qkv + (long long)b * p.qkv_ld + (long long)(hk * p.G + g) * D);
        rope_rotate_pieces(__ldg(src + c), __ldg(src + c2), __ldg(cr + c), __ldg(sr + c), o1, o2);
      }
      *reinterpret_cast<uint4*>(sQ + (c / 8) * (kNPad * 128) + sw128_offset(g, c % 8)) = o1;
      *reinterpret_cast<uint4*>(sQ + (c2 / 8) * (kNPad * 128) + sw128_offset(g, c2 % 8)) = o2;
    }
  } else {
    constexpr int kChunksPerRow = D / 8;  // 16-byte chunks
    for (int i = tid; i < GT * kChunksPerRow; i += 128) {
      const int g = i / kChunksPerRow, c = i % kChunksPerRow;
      uint4 v = make_uint4(0, 0, 0, 0);
      if (g < p.G)
        v = __ldg(reinterpret_cast<const uint4*>(p.q + ((long long)b * p.Hq + hk * p.G + g) * D) + c);
      const int box = c / 8, cc = c % 8;
      *reinterpret_cast<uint4*>(sQ + box * (kNPad * 128) + sw128_offset(g, cc)) = v;
    }
  }
  if (D == 64) {  // zero pad standing in for V dims 64..127
    for (int i = tid; i < SM::kHalfBytes / 16; i += 128)
      reinterpret_cast<uint4*>(sV + SM::kHalfBytes)[i] = make_uint4(0, 0, 0, 0);
  }
  fence_proxy_async_smem();
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  pdl_trigger();  // tensor memory is allocated: the next kernel may be scheduled
  const uint32_t tmem_s = tmem_base;        // columns [0, 16)
  const uint32_t tmem_o = tmem_base + 16;   // columns [16, 32)

  // Running log-sum-exp merge of this CTA's chunks: thread d keeps O^T[d, g] for its head
  // dimension d; every thread keeps the running maximum and denominator of every head.
  float m_run[GT], l_run[GT], o_acc[GT];
#pragma unroll
  for (int g = 0; g < GT; ++g) m_run[g] = -INFINITY, l_run[g] = 0.0f, o_acc[g] = 0.0f;

  // A CTA walks chunks first, first + stride, ...: the next chunk's K tile is requested as soon
  // as S^T has been computed from the current one, and its V tile as soon as O^T has, so loads
  // stay in flight under the softmax / second-MMA tail.  Every barrier completes once per
  // iteration: parity = iteration & 1.
  bool ok = true;
  uint32_t ph = 0;
  RopeRow<kRotate ? D : 16> rope;  // (a one-piece dummy when K is stored rotated)
  if constexpr (kRotate) load_rope_row<D>(rope, p, (c_lo + first) * kChunk, min(kChunk, L - (c_lo + first) * kChunk));
  for (int chunk = c_lo + first; chunk < n_chunks; chunk += stride, ph ^= 1) {
    const int tok0 = chunk * kChunk;
    const int valid = min(kChunk, L - tok0);
    const int next = chunk + stride;

    const bool has_new = append && chunk == c_new;  // (uniform over the CTA)
    if constexpr (kRotate) {
      ok = mbar_wait(bar_k, ph, abort_flag, p.d_status, XAXB_DEVICE_TIMEOUT * 1000 + kSiteDecK);
      if (has_new) {  // the un-rotated new key goes in first; other threads rotate its row below
        if (ok) place_new_key<D>(sK, p, b, hk, t_new, r_new);
        __syncthreads();
      }
      if (ok) rotate_k_row<D>(sK, rope);
      fence_proxy_async_smem();
      ok = __syncthreads_and(ok);
      if (!ok) break;
      // the table rows of the next tile, requested a whole iteration before they are needed
      if (next < n_chunks) load_rope_row<D>(rope, p, next * kChunk, min(kChunk, L - next * kChunk));
    } else if (has_new) {
      ok = mbar_wait(bar_k, ph, abort_flag, p.d_status, XAXB_DEVICE_TIMEOUT * 1000 + kSiteDecK);
      if (ok) place_new_key<D>(sK, p, b, hk, t_new, r_new);
      fence_proxy_async_smem();
      ok = __syncthreads_and(ok);
      if (!ok) break;
    }

    // ---- S^T = K Q^T ---------------------------------------------------------------------
    if (tid == 0) {
      if (mbar_wait(bar_k, ph, abort_flag, p.d_status, XAXB_DEVICE_TIMEOUT * 1000 + kSiteDecK)) {
        tc_fence_after_sync();
        constexpr uint32_t idesc = umma_idesc(kFmtBF16, kFmtBF16, 0, 0, 128, kNPad);
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {  // 16 bf16 = 32 bytes of K per MMA
          const uint32_t box = k / 4, off = (k % 4) * 32;
          const uint64_t a_desc = umma_desc_kmajor_sw128(smem_u32(sK + box * SM::kHalfBytes) + off);
          const uint64_t b_desc = umma_desc_kmajor_sw128(smem_u32(sQ + box * (kNPad * 128)) + off);
          umma_f16(tmem_s, a_desc, b_desc, idesc, k != 0);
        }
        umma_commit(bar_s);
      }
    }
    ok = mbar_wait(bar_s, ph, abort_flag, p.d_status, XAXB_DEVICE_TIMEOUT * 1000 + kSiteDecS);
    if (tid == 0 && ok && next < n_chunks)  // the K tile has been consumed: fetch the next one
      load_tile<D>(sK, &tmap_k, &tmap_k_part, bar_k, hk, next * kChunk, b, min(kChunk, L - next * kChunk));

    // ---- softmax numerators: thread = token ------------------------------------------------
    float pvals[GT];
    if (ok) {
      tc_fence_after_sync();
      uint32_t r[16];
      tmem_ld_x16(tmem_s + (uint32_t(warp * 32) << 16), r);
      tmem_ld_wait();
      tc_fence_before_sync();
      const bool tok_ok = tid < valid && tok0 + tid >= lo_tok;
#pragma unroll
      for (int g = 0; g < GT; ++g) {
        pvals[g] = tok_ok ? __uint_as_float(r[g]) * p.sm_scale : -INFINITY;
        const float wm = warp_max_f32(pvals[g]);
        if (lane == 0) red_max[warp * kNPad + g] = wm;
      }
    }
    ok = __syncthreads_and(ok);
    if (!ok) break;
    float m_c[GT];
    {
      // P^T as the B operand: row g, 128 tokens (two 64-token boxes), K-major, swizzled.
      const int box = tid / 64, within = tid % 64;
#pragma unroll
      for (int g = 0; g < GT; ++g) {
        m_c[g] = fmaxf(fmaxf(red_max[g], red_max[kNPad + g]), fmaxf(red_max[2 * kNPad + g], red_max[3 * kNPad + g]));
        const float e = (tid < valid && tok0 + tid >= lo_tok) ? __expf(pvals[g] - m_c[g]) : 0.0f;
        pvals[g] = e;
        const uint32_t off = box * (kNPad * 128) + sw128_offset(g, within / 8) + (within % 8) * 2;
        *reinterpret_cast<__nv_bfloat16*>(sP + off) = __float2bfloat16_rn(e);
      }
    }
    ok = mbar_wait(bar_v, ph, abort_flag, p.d_status, XAXB_DEVICE_TIMEOUT * 1000 + kSiteDecV);
    if (ok && tid >= valid) {
      // rows past the sequence end may hold anything: clear them so 0 * garbage stays 0
#pragma unroll
      for (int c = 0; c < D / 8; ++c)
        *reinterpret_cast<uint4*>(sV + (c / 8) * SM::kHalfBytes + sw128_offset(tid, c % 8)) = make_uint4(0, 0, 0, 0);
    }
    if (ok && has_new) place_new_value<D>(sV, p, b, hk, t_new, r_new);
    fence_proxy_async_smem();
    ok = __syncthreads_and(ok);
    if (!ok) break;

    // ---- O^T = V^T P ---------------------------------------------------------------------
    if (tid == 0) {
      tc_fence_after_sync();
      constexpr uint32_t idesc = umma_idesc(kFmtBF16, kFmtBF16, 1, 0, 128, kNPad);
#pragma unroll
      for (int k = 0; k < kChunk / 16; ++k) {  // 16 tokens per MMA
        const uint64_t a_desc = umma_desc_mnmajor_sw128(smem_u32(sV) + k * 16 * 128, SM::kHalfBytes);
        const uint64_t b_desc = umma_desc_kmajor_sw128(smem_u32(sP + (k / 4) * (kNPad * 128)) + (k % 4) * 32);
        umma_f16(tmem_o, a_desc, b_desc, idesc, k != 0);
      }
      umma_commit(bar_o);
    }
    // The denominators are reduced while the second MMA runs.
#pragma unroll
    for (int g = 0; g < GT; ++g) {
      float s = pvals[g];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
      if (lane == 0) red_sum[warp * kNPad + g] = s;
    }
    __syncthreads();
    float wa[GT], wb[GT];  // weights of the running state and of this chunk in the merged state
#pragma unroll
    for (int g = 0; g < GT; ++g) {
      const float l_c = red_sum[g] + red_sum[kNPad + g] + red_sum[2 * kNPad + g] + red_sum[3 * kNPad + g];
      const float m_new = fmaxf(m_run[g], m_c[g]);  // m_c is finite: every chunk has a valid token
      wa[g] = __expf(m_run[g] - m_new);
      wb[g] = __expf(m_c[g] - m_new);
      l_run[g] = l_run[g] * wa[g] + l_c * wb[g];
      m_run[g] = m_new;
    }
    ok = mbar_wait(bar_o, ph, abort_flag, p.d_status, XAXB_DEVICE_TIMEOUT * 1000 + kSiteDecO);
    if (tid == 0 && ok && next < n_chunks)  // the V tile has been consumed: fetch the next one
      load_tile<D>(sV, &tmap_v, &tmap_v_part, bar_v, hk, next * kChunk, b, min(kChunk, L - next * kChunk));
    if (ok) {
      tc_fence_after_sync();
      // accumulator row d (a head dimension) sits in TMEM lane d
      uint32_t r[16];
      tmem_ld_x16(tmem_o + (uint32_t(warp * 32) << 16), r);
      tmem_ld_wait();
      tc_fence_before_sync();
#pragma unroll
      for (int g = 0; g < GT; ++g) o_acc[g] = o_acc[g] * wa[g] + __uint_as_float(r[g]) * wb[g];
    }
    // A thread whose wait gave up leaves with everyone else at the next barrier it shares.
  }
  ok = __syncthreads_and(ok);
  if (ok) {
    // One partial result per CTA, in slot `first` of the (sequence, head)'s row of the workspace.
    const int d = tid;
#pragma unroll
    for (int g = 0; g < GT; ++g) {
      if (g < p.G) {
        const long long slot = ((long long)b * p.Hq + hk * p.G + g) * p.max_chunks + first;
        if (d < D) p.ws_o[slot * D + d] = o_acc[g];
        if (tid == g) {
          p.ws_ml[slot * 2 + 0] = m_run[g];
          p.ws_ml[slot * 2 + 1] = l_run[g];
        }
      }
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 32);
  }
}

static int g_decode_variant = 0;  // 0 / 1 = automatic choice of chunks per CTA, 10 + n = n chunks per CTA

// Merge the partial results of one (sequence, query head): out = sum_c w_c O_c / sum_c w_c l_c
// with w_c = exp(m_c - max m).  A sequence of n chunks has min(n, lanes) partial results, in the
// first slots of its row of the workspace.  D threads.
__global__ void attn_decode_merge_kernel(const float* __restrict__ ws_o, const float* __restrict__ ws_ml,
                                         const int32_t* __restrict__ positions, int Hq, int D, int max_chunks,
                                         int lanes, int window, __nv_bfloat16* __restrict__ out) {
  pdl_trigger();
  pdl_wait();
  const int h = blockIdx.x, b = blockIdx.y, d = threadIdx.x;
  const int L = min(max(positions[b] + 1, 1), max_chunks * kChunk);  // clamped like the attention kernel
  const int n = min(decode_chunks(L, window), lanes);
  const long long base = ((long long)b * Hq + h) * max_chunks;
  float m = -INFINITY;
  for (int c = 0; c < n; ++c) m = fmaxf(m, ws_ml[(base + c) * 2]);
  float num = 0.0f, den = 0.0f;
  for (int c = 0; c < n; ++c) {
    const float w = __expf(ws_ml[(base + c) * 2] - m);
    num = fmaf(w, ws_o[(base + c) * D + d], num);
    den = fmaf(w, ws_ml[(base + c) * 2 + 1], den);
  }
  // (times the reciprocal, as the merge + cast pass and the prefill kernel normalise: the three agree bit for bit)
  out[((long long)b * Hq + h) * D + d] = __float2bfloat16_rn(num * (1.0f / den));
}

// Merge + per-token cast as a kernel of its own: one CTA of 512 threads per sequence, one work item
// (a head's 8 consecutive dimensions) per thread -- with one CTA per SM the kernel is bound by the
// latency of each thread's own instruction stream, so the stream is kept short.
__global__ void __launch_bounds__(512) attn_decode_merge_cast_kernel(
    const float* __restrict__ ws_o, const float* __restrict__ ws_ml, const int32_t* __restrict__ positions, int Hq,
    int D, int max_chunks, int lanes, int window, const MergeOut mo, const TpRowMax tp, int* d_status) {
  pdl_trigger();
  pdl_wait();
  __shared__ float s_max[64], s_inv_den[64];
  __shared__ uint32_t s_tp[2];
  const int b = blockIdx.x;
  const int L = min(max(positions[b] + 1, 1), max_chunks * kChunk);  // clamped like the attention kernel
  const int n = min(decode_chunks(L, window), lanes);
  merge_cast_row<512, false>(ws_o, ws_ml, b, n, Hq, D, max_chunks, mo, tp, d_status, s_max, s_inv_den, s_tp);
}

static int make_cache_tmap(const Ctx* ctx, CUtensorMap* map, const void* cache, int64_t B, int64_t max_len,
                           int64_t Hkv, int64_t D, int box_rows = kChunk) {
  // cache[b][token][head][d]: dims innermost first (d, head, token, b); box = 64 d x 1 head x box_rows tokens x 1.
  const uint64_t dims[4] = {(uint64_t)D, (uint64_t)Hkv, (uint64_t)max_len, (uint64_t)B};
  const uint64_t strides[3] = {(uint64_t)D * 2, (uint64_t)Hkv * D * 2, (uint64_t)max_len * Hkv * D * 2};
  const uint32_t box[4] = {64, 1, (uint32_t)box_rows, 1};
  return make_tmap_4d(ctx, map, cache, 2, dims, strides, box);
}

}  // namespace xaxb

using namespace xaxb;

extern "C" {

int64_t xaxb_attn_decode_workspace_bytes(int64_t B, int64_t Hq, int64_t D, int64_t max_len) {
  const int64_t chunks = (max_len + kChunk - 1) / kChunk;
  return B * Hq * chunks * (D + 2) * (int64_t)sizeof(float);
}

static int decode_launch(xaxb_ctx* ctx_, void* stream, const void* q_rot_bf16, const void* k_cache_bf16,
                         const void* v_cache_bf16, const int32_t* positions, int64_t B, int64_t Hq, int64_t Hkv,
                         int64_t D, int64_t max_len, float softmax_scale, int k_is_rotated, const void* cos_bf16,
                         const void* sin_bf16, int64_t table_len, void* out_bf16, void* q_e4m3, float* row_scale,
                         float* row_inv_scale, void* workspace, int64_t workspace_bytes,
                         const TpRowMax* tp = nullptr, int64_t window = -1, const void* qkv_bf16 = nullptr,
                         int64_t qkv_ld = 0) {
  // qkv_bf16: fused append (DecodeParams::qkv); q_rot_bf16 is then unused and the caches are written
  if (!ctx_ || (!q_rot_bf16 && !qkv_bf16) || !k_cache_bf16 || !v_cache_bf16 || !positions || (!out_bf16 && !q_e4m3) ||
      !workspace || B <= 0 || Hq <= 0 || Hkv <= 0 || max_len <= 0) {
    set_last_error("attn_decode: null pointer or non-positive shape");
    return XAXB_BAD_ARGUMENT;
  }
  if (qkv_bf16 && (!cos_bf16 || !sin_bf16 || table_len < max_len || qkv_ld < (Hq + 2 * Hkv) * D || qkv_ld % 8 != 0 ||
                   (reinterpret_cast<uintptr_t>(qkv_bf16) & 15) || (reinterpret_cast<uintptr_t>(cos_bf16) & 15) ||
                   (reinterpret_cast<uintptr_t>(sin_bf16) & 15))) {
    set_last_error("attn_decode_append: needs cos/sin tables covering max_len, a row stride of at least "
                   "(Hq + 2 Hkv) * D that is a multiple of 8, and 16-byte aligned qkv / tables");
    return XAXB_BAD_ARGUMENT;
  }
  if (Hq % Hkv != 0 || Hq / Hkv > kNPad || (D != 128 && D != 64) || Hkv > 65535 || B > 65535) {
    set_last_error("attn_decode: needs head_dim 64 or 128 and at most %d query heads per kv head", kNPad);
    return XAXB_UNSUPPORTED;
  }
  if (!k_is_rotated && (!cos_bf16 || !sin_bf16 || table_len < max_len)) {
    set_last_error("attn_decode: rotate-on-load needs cos/sin tables covering max_len");
    return XAXB_BAD_ARGUMENT;
  }
  if (workspace_bytes < xaxb_attn_decode_workspace_bytes(B, Hq, D, max_len)) return XAXB_WORKSPACE_TOO_SMALL;
  if (reinterpret_cast<uintptr_t>(q_rot_bf16) & 15) return XAXB_BAD_ARGUMENT;
  if (!k_is_rotated && ((reinterpret_cast<uintptr_t>(cos_bf16) | reinterpret_cast<uintptr_t>(sin_bf16)) & 15))
    return XAXB_BAD_ARGUMENT;
  const Ctx* ctx = reinterpret_cast<const Ctx*>(ctx_);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  CUtensorMap tk, tv;
  int rc = make_cache_tmap(ctx, &tk, k_cache_bf16, B, max_len, Hkv, D);
  if (rc) return rc;
  rc = make_cache_tmap(ctx, &tv, v_cache_bf16, B, max_len, Hkv, D);
  if (rc) return rc;
  CUtensorMap tkp, tvp;  // the same caches in boxes of kPartRows token rows, for partly filled chunks
  rc = make_cache_tmap(ctx, &tkp, k_cache_bf16, B, max_len, Hkv, D, kPartRows);
  if (rc) return rc;
  rc = make_cache_tmap(ctx, &tvp, v_cache_bf16, B, max_len, Hkv, D, kPartRows);
  if (rc) return rc;
  const int max_chunks = (int)((max_len + kChunk - 1) / kChunk);
  DecodeParams p;
  p.q = static_cast<const __nv_bfloat16*>(q_rot_bf16);
  p.positions = positions;
  p.Hq = (int)Hq, p.Hkv = (int)Hkv, p.G = (int)(Hq / Hkv);
  p.max_len = max_len;
  p.sm_scale = softmax_scale;
  p.k_is_rotated = k_is_rotated;
  p.cos_t = static_cast<const __nv_bfloat16*>(cos_bf16);
  p.sin_t = static_cast<const __nv_bfloat16*>(sin_bf16);
  p.table_len = table_len;
  p.ws_o = static_cast<float*>(workspace);
  p.ws_ml = p.ws_o + B * Hq * max_chunks * D;
  p.max_chunks = max_chunks;
  p.window = window < 0 ? -1 : (window > 0x3fffffff ? 0x3fffffff : (int)window);
  p.d_status = ctx->d_status;
  p.qkv = static_cast<const __nv_bfloat16*>(qkv_bf16);
  p.qkv_ld = qkv_ld;
  p.k_cache = static_cast<__nv_bfloat16*>(const_cast<void*>(k_cache_bf16));  // written only with qkv set
  p.v_cache = static_cast<__nv_bfloat16*>(const_cast<void*>(v_cache_bf16));
  int lanes = max_chunks;  // partial results per (sequence, head) row of the workspace
  {
    // Chunks are dealt to `lanes` CTAs per (sequence, kv head); each CTA walks its chunks with
    // the next tile's loads in flight.  About seven chunks per CTA: long walks amortise a CTA's set-up
    // and leave fewer partial results to merge, short ones balance the SMs.  Measured (attention +
    // merge): B = 128, 8 kv heads, 17 of 20 chunks: 1 / 2-4 / 5 / 7 / 10 lanes 175 / 171 / 173 / 175 /
    // 177 us; the ragged B = 32 case of 4 - 64 chunks: 2 / 4 / 8 / 16 lanes 103.5 / 101.4 / 99.3 /
    // 103.3 us; B = 64, 4 kv heads, 5 of 6 chunks: 1 / 2 / 3 / 6 lanes 20.2 / 23.0 / 22.9 / 25.7 us.
    // With fewer (sequence, head) groups than SMs the lanes are raised so that every SM has a CTA.
    const long long groups = (long long)B * Hkv;
    lanes = (max_chunks + 6) / 7;
    if (groups * lanes < ctx->num_sms) lanes = (int)((ctx->num_sms + groups - 1) / groups);
    if (g_decode_variant >= 11) {  // test hook: a fixed number of chunks per CTA
      const int per_cta = g_decode_variant - 10;
      lanes = (max_chunks + per_cta - 1) / per_cta;
    }
    if (lanes > max_chunks) lanes = max_chunks;
    if (lanes < 1) lanes = 1;
    dim3 grid((unsigned)lanes, (unsigned)Hkv, (unsigned)B);
    const int G = p.G;
    const int gt = G <= 1 ? 1 : G <= 2 ? 2 : G <= 4 ? 4 : G <= 8 ? 8 : 16;
#define XAXB_DECODE_CASE(DD, GG)                                                                                 \
  if (D == DD && gt == GG) {                                                                                     \
    if (k_is_rotated) {                                                                                          \
      rc = ensure_dynamic_smem<attn_decode_kernel<DD, GG, false>>(ctx, DecodeSmem<DD>::kBytes, "attn_decode");   \
      if (rc) return rc;                                                                                         \
      launch_kernel(attn_decode_kernel<DD, GG, false>, grid, dim3(128), DecodeSmem<DD>::kBytes, s, 1, tk, tv, tkp, tvp, p);\
    } else {                                                                                                     \
      rc = ensure_dynamic_smem<attn_decode_kernel<DD, GG, true>>(ctx, DecodeSmem<DD>::kBytes, "attn_decode");    \
      if (rc) return rc;                                                                                         \
      launch_kernel(attn_decode_kernel<DD, GG, true>, grid, dim3(128), DecodeSmem<DD>::kBytes, s, 1, tk, tv, tkp, tvp, p); \
    }                                                                                                            \
  }
    XAXB_DECODE_CASE(128, 1) XAXB_DECODE_CASE(128, 2) XAXB_DECODE_CASE(128, 4) XAXB_DECODE_CASE(128, 8)
    XAXB_DECODE_CASE(128, 16) XAXB_DECODE_CASE(64, 1) XAXB_DECODE_CASE(64, 2) XAXB_DECODE_CASE(64, 4)
    XAXB_DECODE_CASE(64, 8) XAXB_DECODE_CASE(64, 16)
#undef XAXB_DECODE_CASE
  }
  rc = check_launch("attn_decode_kernel");
  if (rc) return rc;
  if (q_e4m3) {
    launch_kernel(attn_decode_merge_cast_kernel, dim3((unsigned)B), dim3(512), 0, s, 1, p.ws_o, p.ws_ml, positions, (int)Hq, (int)D, max_chunks,
                                                             lanes, p.window,
                  MergeOut{static_cast<uint4*>(out_bf16), static_cast<uint2*>(q_e4m3), row_scale, row_inv_scale},
                  tp ? *tp : TpRowMax{}, ctx->d_status);
    return check_launch("attn_decode_merge_cast_kernel");
  }
  dim3 mgrid((unsigned)Hq, (unsigned)B);
  launch_kernel(attn_decode_merge_kernel, mgrid, dim3((unsigned)D), 0, s, 1, p.ws_o, p.ws_ml, positions, (int)Hq, (int)D, max_chunks,
                                                         lanes, p.window, static_cast<__nv_bfloat16*>(out_bf16));
  return check_launch("attn_decode_merge_kernel");
}

int xaxb_attn_decode(xaxb_ctx* ctx_, void* stream, const void* q_rot_bf16, const void* k_cache_bf16,
                     const void* v_cache_bf16, const int32_t* positions, int64_t B, int64_t Hq, int64_t Hkv, int64_t D,
                     int64_t max_len, float softmax_scale, int k_is_rotated, const void* cos_bf16,
                     const void* sin_bf16, int64_t table_len, void* out_bf16, void* workspace,
                     int64_t workspace_bytes) {
  if (!out_bf16) return XAXB_BAD_ARGUMENT;
  return decode_launch(ctx_, stream, q_rot_bf16, k_cache_bf16, v_cache_bf16, positions, B, Hq, Hkv, D, max_len,
                       softmax_scale, k_is_rotated, cos_bf16, sin_bf16, table_len, out_bf16, nullptr, nullptr, nullptr,
                       workspace, workspace_bytes);
}

int xaxb_attn_decode_window(xaxb_ctx* ctx_, void* stream, const void* q_rot_bf16, const void* k_cache_bf16,
                            const void* v_cache_bf16, const int32_t* positions, int64_t B, int64_t Hq, int64_t Hkv,
                            int64_t D, int64_t max_len, float softmax_scale, int64_t window, void* out_bf16,
                            void* workspace, int64_t workspace_bytes) {
  if (!out_bf16) return XAXB_BAD_ARGUMENT;
  return decode_launch(ctx_, stream, q_rot_bf16, k_cache_bf16, v_cache_bf16, positions, B, Hq, Hkv, D, max_len,
                       softmax_scale, 1, nullptr, nullptr, 0, out_bf16, nullptr, nullptr, nullptr, workspace,
                       workspace_bytes, nullptr, window);
}

int xaxb_attn_decode_cast(xaxb_ctx* ctx_, void* stream, const void* q_rot_bf16, const void* k_cache_bf16,
                          const void* v_cache_bf16, const int32_t* positions, int64_t B, int64_t Hq, int64_t Hkv,
                          int64_t D, int64_t max_len, float softmax_scale, int k_is_rotated, const void* cos_bf16,
                          const void* sin_bf16, int64_t table_len, void* out_bf16, void* q_e4m3, float* row_scale,
                          float* row_inv_scale, void* workspace, int64_t workspace_bytes) {
  if (!q_e4m3 || !row_scale || !row_inv_scale) return XAXB_BAD_ARGUMENT;
  if (Hq > 64 || Hq * D > 4096 || (reinterpret_cast<uintptr_t>(q_e4m3) & 7) ||
      (reinterpret_cast<uintptr_t>(out_bf16) & 15)) {
    set_last_error("attn_decode_cast: needs Hq <= 64, Hq * D <= 4096 and aligned outputs");
    return XAXB_UNSUPPORTED;
  }
  return decode_launch(ctx_, stream, q_rot_bf16, k_cache_bf16, v_cache_bf16, positions, B, Hq, Hkv, D, max_len,
                       softmax_scale, k_is_rotated, cos_bf16, sin_bf16, table_len, out_bf16, q_e4m3, row_scale,
                       row_inv_scale, workspace, workspace_bytes);
}

}  // extern "C"

// ---------------------------------------------------------------------------------------
// Allocation-free variant of decode attention.
//
// Some callers cannot obtain device memory at the point where they run attention: code
// that executes inside a framework's custom-call handler where only the buffers declared
// up front exist, real-time serving loops that forbid cudaMalloc because it synchronises
// the device, and embedders that own the allocator and hand this library nothing but input
// and output pointers.  For them the per-chunk partial results live in a fixed array that is
// part of the loaded library image instead of a caller-provided workspace.
//
// The array costs every GPU that loads the library kStaticScratchBytes of device memory until
// the process exits.  It is shared by all calls and keeps whatever the previous call left in
// it; the decode kernel writes every slot it later reads, so nothing needs clearing.  Two
// calls that overlap on the GPU (different streams) would write the same slots: callers must
// serialise them.

namespace xaxb {

constexpr long long kStaticScratchBytes = 16ll << 20;  // 16 MiB per GPU
constexpr int kMaxDevices = 64;

static __device__ __align__(256) unsigned char g_decode_scratch[kStaticScratchBytes];

// Device address of g_decode_scratch per device ordinal.  In host code the array's name is
// only a handle for the runtime, not an address a kernel could use, so the address is looked
// up once per device (with that device current) and cached.
static void* g_decode_scratch_addr[kMaxDevices] = {nullptr};

}  // namespace xaxb

extern "C" int xaxb_attn_decode_cast_tp(xaxb_ctx* ctx_, void* stream, const void* q_rot_bf16, const void* k_cache_bf16,
                             const void* v_cache_bf16, const int32_t* positions, int64_t B, int64_t Hq, int64_t Hkv,
                             int64_t D, int64_t max_len, float softmax_scale, int k_is_rotated, const void* cos_bf16,
                             const void* sin_bf16, int64_t table_len, void* q_e4m3, float* row_scale,
                             float* row_inv_scale, void* workspace, int64_t workspace_bytes, void* const* peer_bases,
                             int rank, int world, int64_t inbox_offset_bytes, int64_t sync_offset_bytes) {
  if (!q_e4m3 || !row_scale || !row_inv_scale) return XAXB_BAD_ARGUMENT;
  if (Hq > 64 || Hq * D > 4096 || B > xaxb::kTpMaxSlots || (reinterpret_cast<uintptr_t>(q_e4m3) & 7)) {
    set_last_error("attn_decode_cast_tp: needs Hq <= 64, Hq * D <= 4096, B <= %d and an aligned output",
                   xaxb::kTpMaxSlots);
    return XAXB_UNSUPPORTED;
  }
  xaxb::TpRowMax tp;
  int rc = xaxb::fill_tp_rowmax(tp, peer_bases, rank, world, inbox_offset_bytes, sync_offset_bytes,
                                "attn_decode_cast_tp");
  if (rc) return rc;
  return decode_launch(ctx_, stream, q_rot_bf16, k_cache_bf16, v_cache_bf16, positions, B, Hq, Hkv, D, max_len,
                       softmax_scale, k_is_rotated, cos_bf16, sin_bf16, table_len, nullptr, q_e4m3, row_scale,
                       row_inv_scale, workspace, workspace_bytes, &tp);
}

extern "C" int xaxb_attn_decode_append(xaxb_ctx* ctx_, void* stream, const void* qkv_bf16, int64_t ld, void* k_cache_bf16,
                                       void* v_cache_bf16, const int32_t* positions, int64_t B, int64_t Hq,
                                       int64_t Hkv, int64_t D, int64_t max_len, float softmax_scale,
                                       int k_is_rotated, const void* cos_bf16, const void* sin_bf16,
                                       int64_t table_len, int64_t window, void* out_bf16, void* q_e4m3,
                                       float* row_scale, float* row_inv_scale, void* workspace,
                                       int64_t workspace_bytes, void* const* peer_bases, int rank, int world,
                                       int64_t inbox_offset_bytes, int64_t sync_offset_bytes) {
  if (!qkv_bf16) return XAXB_BAD_ARGUMENT;
  if (q_e4m3) {
    if (!row_scale || !row_inv_scale) return XAXB_BAD_ARGUMENT;
    if (Hq > 64 || Hq * D > 4096 || (reinterpret_cast<uintptr_t>(q_e4m3) & 7) ||
        (reinterpret_cast<uintptr_t>(out_bf16) & 15)) {
      set_last_error("attn_decode_append: the cast output needs Hq <= 64, Hq * D <= 4096 and aligned outputs");
      return XAXB_UNSUPPORTED;
    }
  }
  xaxb::TpRowMax tp;
  const bool with_tp = peer_bases != nullptr && world > 1;
  if (with_tp) {
    if (!q_e4m3 || B > xaxb::kTpMaxSlots) {
      set_last_error("attn_decode_append: the exchange over ranks needs the cast output and B <= %d", xaxb::kTpMaxSlots);
      return XAXB_UNSUPPORTED;
    }
    int rc = xaxb::fill_tp_rowmax(tp, peer_bases, rank, world, inbox_offset_bytes, sync_offset_bytes,
                                  "attn_decode_append");
    if (rc) return rc;
  }
  return decode_launch(ctx_, stream, nullptr, k_cache_bf16, v_cache_bf16, positions, B, Hq, Hkv, D, max_len,
                       softmax_scale, k_is_rotated, cos_bf16, sin_bf16, table_len, out_bf16, q_e4m3, row_scale,
                       row_inv_scale, workspace, workspace_bytes, with_tp ? &tp : nullptr, window, qkv_bf16, ld);
}

extern "C" int xaxb_attn_decode_force_variant(int variant) {
  if (variant < 0 || (variant > 1 && variant < 11) || variant > 74) return XAXB_BAD_ARGUMENT;
  xaxb::g_decode_variant = variant;
  return XAXB_OK;
}

extern "C" int64_t xaxb_attn_decode_static_capacity_bytes(void) { return xaxb::kStaticScratchBytes; }

extern "C" int xaxb_attn_decode_static(xaxb_ctx* ctx_, void* stream, const void* q_rot_bf16, const void* k_cache_bf16,
                                       const void* v_cache_bf16, const int32_t* positions, int64_t B, int64_t Hq,
                                       int64_t Hkv, int64_t D, int64_t max_len, float softmax_scale, int k_is_rotated,
                                       const void* cos_bf16, const void* sin_bf16, int64_t table_len, void* out_bf16) {
  if (!ctx_) return XAXB_BAD_ARGUMENT;
  const Ctx* ctx = reinterpret_cast<const Ctx*>(ctx_);
  if (B <= 0 || Hq <= 0 || D <= 0 || max_len <= 0) {
    set_last_error("attn_decode_static: non-positive shape");
    return XAXB_BAD_ARGUMENT;
  }
  const int64_t need = xaxb_attn_decode_workspace_bytes(B, Hq, D, max_len);
  if (need > kStaticScratchBytes) {
    set_last_error("attn_decode_static: B=%lld Hq=%lld D=%lld max_len=%lld needs %lld bytes of scratch, the built-in "
                   "array holds %lld; use xaxb_attn_decode with a caller-provided workspace",
                   (long long)B, (long long)Hq, (long long)D, (long long)max_len, (long long)need,
                   (long long)kStaticScratchBytes);
    return XAXB_WORKSPACE_TOO_SMALL;
  }
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= kMaxDevices || dev != ctx->device) {
    set_last_error("attn_decode_static: the context's device (%d) must be current (current: %d)", ctx->device, dev);
    return XAXB_BAD_ARGUMENT;
  }
  if (!g_decode_scratch_addr[dev]) {  // first call on this device: not inside a stream capture
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_decode_scratch);
    if (e != cudaSuccess || !p) {
      set_last_error("attn_decode_static: cudaGetSymbolAddress: %s", cudaGetErrorString(e));
      return XAXB_LAUNCH_FAILED;
    }
    g_decode_scratch_addr[dev] = p;
  }
  return xaxb_attn_decode(ctx_, stream, q_rot_bf16, k_cache_bf16, v_cache_bf16, positions, B, Hq, Hkv, D, max_len,
                          softmax_scale, k_is_rotated, cos_bf16, sin_bf16, table_len, out_bf16,
                          g_decode_scratch_addr[dev], kStaticScratchBytes);
}
