// Next-token choice with temperature, nucleus (top-p) truncation and the generation loop's token
// masks, without sorting the vocabulary.
//
// The reference sorts the scaled logits, takes a softmax and a cumulative sum over the sorted
// order, keeps the tokens whose inclusive cumulative probability does not exceed top_p (the first
// always) and draws from the kept ones (xax/arch/llm.py:1446-1489).  bf16 logits take at most 65536
// distinct values, and tokens with equal logits are neighbours in the sorted order (ties keep index
// order), so everything the sort is used for can be answered from
//     mass_ge(k) = sum of exp((l_i - l_max) / T) over tokens whose logit, as an order-preserving
//                  16-bit key, is >= k,
// evaluated by a deterministic block reduction over the row:
//   * the kept set is every level (key value) k with mass_ge(k) <= top_p * Z, found by bisection on
//     k, plus the first n_b tokens (by index) of the next level down, n_b from the level's
//     per-token weight;
//   * the draw is the inverse CDF over the kept tokens in sorted order at a caller-supplied uniform
//     u: bisection for the level where the running mass crosses u * (kept mass), then the rank inside
//     that level, then a rank-select by index.
// The reference draws through jax.random.categorical (Gumbel noise from its own PRNG stream); the
// distribution is the same, the stream is not reproducible outside JAX, so the uniforms are an input.
//
// One CTA of 1024 threads per row; about forty passes over the row, which stays in L2.
#include "common.cuh"
#include "quant_device.cuh"

namespace xaxb {

constexpr int kSampleThreads = 1024;

struct SampleParams {
  const __nv_bfloat16* logits;
  long long ld;
  int vocab;
  float temperature, top_p;
  const float* uniforms;
  int allowed_min, allowed_max;  // [min, max); allowed_min < 0: no range
  int eos_id, allow_eos;
  int32_t* out;
};

// The generation loop's mask (xax/arch/llm.py:1547-1570).
__device__ __forceinline__ bool token_allowed(const SampleParams& p, int i) {
  if (p.allowed_min < 0) return !(p.eos_id >= 0 && !p.allow_eos && i == p.eos_id);
  const bool in_range = i >= p.allowed_min && i < p.allowed_max;
  return in_range || (p.eos_id >= 0 && p.allow_eos && i == p.eos_id);
}

// Order-preserving 16-bit key of a bf16 value: larger key <=> larger value (NaN with the sign bit
// clear sorts above +inf, as the largest, which is how jnp.argmax treats it).
__device__ __forceinline__ uint32_t bf16_key(uint32_t bits) {
  return (bits & 0x8000u) ? (~bits & 0xFFFFu) : (bits | 0x8000u);
}
__device__ __forceinline__ float key_value(uint32_t key) {
  const uint32_t bits = (key & 0x8000u) ? (key & 0x7FFFu) : (~key & 0xFFFFu);
  return bf16_bits_to_float(bits);
}

constexpr uint32_t kMaskedKey = 0x0080u;  // key of finfo(bfloat16).min = 0xFF7F: what a masked logit is set to

__device__ __forceinline__ uint32_t row_key(const SampleParams& p, const __nv_bfloat16* row, int i) {
  return token_allowed(p, i) ? bf16_key(__bfloat16_as_ushort(row[i])) : kMaskedKey;
}

__device__ __forceinline__ int block_sum_i32(int v) {
  __shared__ int warp_vals[32];
  __shared__ int result;
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();
  if (lane == 0) warp_vals[warp] = v;
  __syncthreads();
  if (warp == 0) {
    int w = lane < (int)((blockDim.x + 31) >> 5) ? warp_vals[lane] : 0;
    for (int o = 16; o > 0; o >>= 1) w += __shfl_xor_sync(0xffffffffu, w, o);
    if (lane == 0) result = w;
  }
  __syncthreads();
  return result;
}

// sum of w(key_i) over tokens with key_i >= t; every thread gets the same value, and the same value
// on every run (fixed order of additions).
__device__ __forceinline__ float mass_ge(const SampleParams& p, const __nv_bfloat16* row, uint32_t t, float s_max,
                                         float inv_t) {
  float acc = 0.0f;
  for (int i = threadIdx.x; i < p.vocab; i += kSampleThreads) {
    const uint32_t k = row_key(p, row, i);
    if (k >= t) acc += __expf(key_value(k) * inv_t - s_max);
  }
  return block_sum_f32(acc);
}

__global__ void __launch_bounds__(kSampleThreads) sample_top_p_kernel(const SampleParams p) {
  pdl_trigger();
  pdl_wait();
  const int r = blockIdx.x;
  const __nv_bfloat16* row = p.logits + (long long)r * p.ld;
  __shared__ int s_pick;

  // ---- the largest key, and the lowest index that holds it
  uint32_t km = 0;
  for (int i = threadIdx.x; i < p.vocab; i += kSampleThreads) km = max(km, row_key(p, row, i));
  const uint32_t kmax = block_max_u32(km);
  if (p.temperature <= 0.0f) {  // greedy: arg-max of the masked logits, first index on ties (:1469-1470, :1489)
    uint32_t best = 0xFFFFFFFFu;
    for (int i = threadIdx.x; i < p.vocab; i += kSampleThreads)
      if (row_key(p, row, i) == kmax) best = min(best, (uint32_t)i);
    const uint32_t first = ~block_max_u32(~best);
    if (threadIdx.x == 0) p.out[r] = (int32_t)first;
    return;
  }
  const float inv_t = 1.0f / p.temperature;
  const float s_max = key_value(kmax) * inv_t;

  // ---- which levels are kept in full: the smallest k with mass_ge(k) <= top_p * Z
  const float Z = mass_ge(p, row, 0u, s_max, inv_t);
  const float P = p.top_p * Z;
  uint32_t k_full = 0;
  float m_full = Z;
  if (!(Z <= P)) {
    uint32_t lo = 0, hi = 65536;  // mass_ge(lo) > P >= mass_ge(hi)
    float m_hi = 0.0f;
    while (hi - lo > 1) {
      const uint32_t mid = (lo + hi) >> 1;
      const float m = mass_ge(p, row, mid, s_max, inv_t);
      if (m > P) lo = mid; else hi = mid, m_hi = m;
    }
    k_full = hi;
    m_full = m_hi;
  }
  // ---- the level below: its first n_b tokens (by index) are kept too
  uint32_t kb_local = 0;
  for (int i = threadIdx.x; i < p.vocab; i += kSampleThreads) {
    const uint32_t k = row_key(p, row, i);
    if (k < k_full) kb_local = max(kb_local, k + 1);
  }
  const uint32_t kb1 = block_max_u32(kb_local);  // boundary key + 1; 0 = no level below
  int n_b = 0;
  float w_b = 0.0f;
  uint32_t kb = 0;
  if (kb1 > 0) {
    kb = kb1 - 1;
    int c = 0;
    for (int i = threadIdx.x; i < p.vocab; i += kSampleThreads) c += row_key(p, row, i) == kb;
    const int c_b = block_sum_i32(c);
    w_b = __expf(key_value(kb) * inv_t - s_max);
    if (w_b > 0.0f) {
      const float room = (P - m_full) / w_b;
      n_b = room <= 0.0f ? 0 : (room >= (float)c_b ? c_b : (int)room);
    }
    if (m_full <= 0.0f && n_b == 0) n_b = 1;  // the first token of the sorted order is always kept (:1479)
  }
  const float kept = m_full + (float)n_b * w_b;

  // ---- inverse CDF over the kept tokens in sorted order
  const float u = fminf(fmaxf(p.uniforms[r], 0.0f), 0.99999994f);
  const float target = u * kept;
  uint32_t ks;
  int rank;
  if (target < m_full) {
    uint32_t lo = k_full, hi = 65536;  // mass_ge(lo) > target >= mass_ge(hi)
    float m_hi = 0.0f;
    while (hi - lo > 1) {
      const uint32_t mid = (lo + hi) >> 1;
      const float m = mass_ge(p, row, mid, s_max, inv_t);
      if (m > target) lo = mid; else hi = mid, m_hi = m;
    }
    ks = lo;
    const float w = __expf(key_value(ks) * inv_t - s_max);
    rank = w > 0.0f ? (int)((target - m_hi) / w) : 0;
  } else {
    ks = kb;
    rank = w_b > 0.0f ? (int)((target - m_full) / w_b) : 0;
    if (rank > n_b - 1) rank = n_b - 1;
  }
  if (rank < 0) rank = 0;

  // ---- the rank-th token (ascending index) at level ks: contiguous slices, a block-wide prefix count
  const int per = (p.vocab + kSampleThreads - 1) / kSampleThreads;
  const int i0 = threadIdx.x * per, i1 = min(p.vocab, i0 + per);
  int cnt = 0;
  for (int i = i0; i < i1; ++i) cnt += row_key(p, row, i) == ks;
  // exclusive prefix over the 1024 threads
  __shared__ int s_warp[32];
  int incl = cnt;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int o = 1; o < 32; o <<= 1) {
    const int n = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += n;
  }
  if (threadIdx.x == 0) s_pick = -1;
  if (lane == 31) s_warp[warp] = incl;
  __syncthreads();
  if (warp == 0) {
    int w = s_warp[lane];
    for (int o = 1; o < 32; o <<= 1) {
      const int n = __shfl_up_sync(0xffffffffu, w, o);
      if (lane >= o) w += n;
    }
    s_warp[lane] = w;  // inclusive over warps
  }
  __syncthreads();
  const int total = s_warp[31];
  if (rank > total - 1) rank = total - 1;
  const int before = (warp ? s_warp[warp - 1] : 0) + incl - cnt;
  if (rank >= before && rank < before + cnt) {
    int left = rank - before;
    for (int i = i0; i < i1; ++i) {
      if (row_key(p, row, i) == ks) {
        if (left == 0) {
          s_pick = i;
          break;
        }
        --left;
      }
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) p.out[r] = s_pick >= 0 ? s_pick : 0;
}

}  // namespace xaxb

using namespace xaxb;

extern "C" int xaxb_sample_top_p(xaxb_ctx* ctx, void* stream, const void* logits_bf16, int64_t rows, int64_t vocab,
                                 int64_t ld, float temperature, float top_p, const float* uniforms,
                                 int32_t allowed_min, int32_t allowed_max, int32_t eos_id, int allow_eos,
                                 int32_t* out) {
  if (!ctx || !logits_bf16 || !out || rows <= 0 || vocab <= 0 || ld < vocab || vocab > 0x7fffffff ||
      (temperature > 0.0f && !uniforms)) {
    set_last_error("sample_top_p: null pointer, non-positive shape, or no uniforms for temperature > 0");
    return XAXB_BAD_ARGUMENT;
  }
  if (allowed_min >= 0 && allowed_max <= allowed_min) {
    set_last_error("sample_top_p: allowed token range must satisfy max > min");
    return XAXB_BAD_ARGUMENT;
  }
  if (!(top_p > 0.0f)) {
    set_last_error("sample_top_p: top_p must be positive");
    return XAXB_BAD_ARGUMENT;
  }
  SampleParams p;
  p.logits = static_cast<const __nv_bfloat16*>(logits_bf16);
  p.ld = ld;
  p.vocab = (int)vocab;
  p.temperature = temperature;
  p.top_p = top_p;
  p.uniforms = uniforms;
  p.allowed_min = allowed_min < 0 ? -1 : allowed_min;
  p.allowed_max = allowed_max;
  p.eos_id = eos_id;
  p.allow_eos = allow_eos;
  p.out = out;
  launch_kernel(sample_top_p_kernel, dim3((unsigned)rows), dim3(kSampleThreads), 0, static_cast<cudaStream_t>(stream),
                1, p);
  return check_launch("sample_top_p_kernel");
}
