/*
 * C ABI of the B200 (sm_100a) kernels behind the xax FP8 transformer inference path.
 *
 * The reference (codekansas/xax) has no FFI layer of its own: its operator interface is
 * the Equinox module API, and XLA picks library kernels at JIT time.  Each entry point
 * below names the reference call site (file:line inside the xax source tree) whose device
 * work it replaces; a `jax.ffi` (or ctypes) binding registers exactly these symbols.
 *
 * Conventions
 *   - every pointer except `ctx`, `stream` and out-parameters of the ctx_* calls is a
 *     DEVICE pointer owned by the caller; no entry point allocates or frees device memory
 *     (xaxb_ctx_create allocates one 32-byte status block, released by xaxb_ctx_destroy);
 *   - `stream` is a cudaStream_t passed as void*; all work is stream-ordered and returns
 *     without synchronising, so calls may be captured in a CUDA graph;
 *   - the return value is an xaxb_status; device-side waits that ran out of time are
 *     reported by xaxb_ctx_status (which synchronises the stream);
 *   - bf16 tensors are row-major with the stated shape; "e4m3" is float8_e4m3fn bytes.
 */
#ifndef XAXB200_H_
#define XAXB200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct xaxb_ctx xaxb_ctx;

typedef enum {
  XAXB_OK = 0,
  XAXB_BAD_ARGUMENT = 1,    /* null pointer, non-positive size, misaligned pointer or stride */
  XAXB_UNSUPPORTED = 2,     /* configuration the kernels do not cover (e.g. head_dim != 64/128) */
  XAXB_WORKSPACE_TOO_SMALL = 3,
  XAXB_LAUNCH_FAILED = 4,   /* CUDA runtime / driver error; see xaxb_last_error */
  XAXB_DEVICE_TIMEOUT = 5,  /* a bounded device-side wait gave up */
  XAXB_CACHE_OVERFLOW = 6   /* position + new tokens > max_len (the reference clamps silently,
                               xax/arch/attention.py:885-888; this library refuses) */
} xaxb_status;

/* ---- context ------------------------------------------------------------------------ */

int xaxb_ctx_create(int device, xaxb_ctx** out);
int xaxb_ctx_destroy(xaxb_ctx* ctx);
/* Synchronises `stream`, returns and clears the device status word (XAXB_OK or
 * XAXB_DEVICE_TIMEOUT with the waiting site in *site, may be NULL). */
int xaxb_ctx_status(xaxb_ctx* ctx, void* stream, int* site);
int xaxb_num_sms(const xaxb_ctx* ctx);
const char* xaxb_status_string(int status);
const char* xaxb_last_error(void);
/* Process-wide switch (default on; off when XAXB_PROGRAMMATIC_LAUNCH=0 is in the environment at
 * load time) for programmatic dependent launch: every kernel of the library is launched so that it
 * may be scheduled while its predecessor in the stream still runs, and waits on the device for that
 * predecessor before touching memory another kernel touches.  Results do not depend on it; 0
 * restores plain stream-ordered launches.  No counterpart in the reference. */
int xaxb_set_programmatic_launch(int on);
int xaxb_programmatic_launch_enabled(void); /* 1 / 0: the switch's current state */
/* Number of kernels this library has launched in the process since the counter was last reset
 * (reset != 0 returns the count and clears it).  Launches recorded into a CUDA graph count once,
 * at capture; replays do not pass through the library.  No counterpart in the reference. */
long long xaxb_launch_count(int reset);
/* Limits of the bounded device-side waits of this context, in milliseconds: `local_ms` for waits
 * inside one GPU (shared-memory barriers fed by TMA / tensor-core completions; default 1000),
 * `peer_ms` for waits on flags that another GPU raises (default 10000).  0 restores the default.
 * A wait that runs out records XAXB_DEVICE_TIMEOUT and its site (xaxb_ctx_status) and the kernel
 * runs to its normal end.  Synchronises with the device.  No counterpart in the reference. */
int xaxb_set_wait_limit_ms(xaxb_ctx* ctx, int local_ms, int peer_ms);

/* ---- kernel 1: amax / scale / e4m3 cast ------------------------------------------- */

/*
 * Current scaling (xax/nn/fp8.py:329-331 + quantize :114-120), one scale per group of
 * `group_rows` consecutive rows of x[rows, cols] (1 = per token, the vmapped call of
 * xax/arch/attention.py:279; rows = per tensor, xax/arch/attention.py:55):
 *     amax_g = max|x_g|                      (bf16, NaN propagates)
 *     s_g    = bf16(448 / max(amax_g, bf16(1e-12)))
 *     q      = e4m3(clip(bf16(x * s_g), +-448))
 * Outputs: q[rows, cols] e4m3; scale[rows] and inv_scale[rows] float32 (s_g and 1/s_g
 * repeated for every row of the group); amax[groups] float32.
 * `amax` doubles as the cross-CTA reduction scratch and is cleared by the call.
 * cols must be a multiple of 8; x and q 16-byte aligned.
 */
int xaxb_quantize_current(xaxb_ctx* ctx, void* stream, const void* x_bf16, int64_t rows, int64_t cols,
                          int64_t group_rows, void* q_e4m3, float* scale, float* inv_scale, float* amax);

/*
 * Delayed scaling (xax/nn/fp8.py:299-326, :82-94, :50-79): quantise with the INCOMING
 * scale *scale_in (float32, rounded to bf16 for the multiply as quantize :117 does), and
 * produce the state for the next call:
 *     history_out = roll(history_in, -1); history_out[0] = max|x|
 *     scale_out   = 448 / max(history_out)   (previous scale kept if that max is <= 0 or
 *                                             not finite)
 * history_in/out float32[history_len] (may alias); amax_scratch: 8 bytes that are zero when
 * the call starts and zero again when it has finished (zero them once; calls that may overlap on
 * the device need a scratch each).  One kernel launch.  q_e4m3 may be NULL to update the state only (used for the weight, whose bytes
 * are quantised once).  inv_scale_out (may be NULL) receives 1 / bf16(*scale_in), the
 * dequantisation multiplier matching the bytes written.
 */
int xaxb_quantize_delayed(xaxb_ctx* ctx, void* stream, const void* x_bf16, int64_t rows, int64_t cols,
                          const float* scale_in, const float* history_in, int history_len, void* q_e4m3,
                          float* history_out, float* scale_out, float* inv_scale_out, float* amax_scratch);

/*
 * Dequantise (xax/nn/fp8.py:123-138): out[r, c] = T(q[r, c]) / T(scale[r * scale_stride]) with T = bfloat16
 * (out_is_bf16 != 0; the quotient rounds once to bf16) or float32; scale_stride 0 = one scale for the tensor,
 * 1 = one per row.  cols a multiple of 8.  The linear layer never calls this (its GEMM consumes the e4m3
 * bytes and applies 1 / scale in the epilogue); it serves the free function of the same name.
 */
int xaxb_dequantize(xaxb_ctx* ctx, void* stream, const void* q_e4m3, int64_t rows, int64_t cols, const float* scale,
                    int scale_stride, int out_is_bf16, void* out);

/*
 * float8_e5m2 for the free functions (xax/nn/fp8.py:97-162 and :347-378 called with fp8_dtype=float8_e5m2; the
 * reference's tests/nn/test_fp8.py parametrises them over both formats).  The transformer path itself quantises
 * to e4m3 only.  x is [rows, cols] bf16, cols a multiple of 8; groups of group_rows rows share a scale, which is
 * either bf16(*scale_in) for every group (quantize with a given scalar scale) or
 * bf16(57344 / max(group_amax[g], bf16(1e-12))) (current scaling; group_amax as xaxb_group_amax leaves it).
 * Exactly one of scale_in / group_amax is non-null.  q = e5m2(clip(bf16(x * s), +-57344)); NaN -> 0x7E / 0xFE.
 * scale / inv_scale ([rows] float32, both or neither) receive s and 1 / s per row.
 */
int xaxb_quantize_e5m2(xaxb_ctx* ctx, void* stream, const void* x_bf16, int64_t rows, int64_t cols, int64_t group_rows,
                       const float* scale_in, const float* group_amax, void* q_e5m2, float* scale, float* inv_scale);

/* xaxb_dequantize for e5m2 bytes (same contract). */
int xaxb_dequantize_e5m2(xaxb_ctx* ctx, void* stream, const void* q_e5m2, int64_t rows, int64_t cols, const float* scale,
                         int scale_stride, int out_is_bf16, void* out);

/* ---- kernel 2: e4m3 x e4m3 (and bf16 x bf16) GEMM on tcgen05 / TMEM ------------- */

/*
 * out[M, N] = bf16( (sum_k a[m,k] * b[n,k]) * row_mul[m] * col_mul[n] + bias[n] + residual[m,n] )
 * replacing x_qdq @ w_qdq.T + bias (xax/nn/fp8.py:339-342) and, with `residual`, the
 * block's x + attn_out / x + ff_out (xax/arch/attention.py:1481,1508).
 * a: e4m3 [M, K] row-major (lda bytes between rows); b: e4m3 [N, K] row-major -- the
 * reference's (out_features, in_features) weight layout; K-contiguous for both.
 * row_mul: float32, element m at row_mul[m * row_mul_stride] (stride 0 = per-tensor scale,
 * 1 = per-token); col_mul likewise over n (stride 0, or 1 for fused projections whose
 * column blocks carry different weight scales).  NULL means 1.0.
 * bias: bf16 [N] or NULL; residual: bf16 [M, N] with ldr elements between rows, or NULL.
 * out: bf16, ldo elements between rows.  K * elem must be a multiple of 16 bytes, a/b
 * 16-byte aligned, N and ldo multiples of 8.
 */
int xaxb_gemm_fp8(xaxb_ctx* ctx, void* stream, const void* a_e4m3, int64_t lda, const void* b_e4m3, int64_t ldb,
                  int64_t M, int64_t N, int64_t K, const float* row_mul, int row_mul_stride, const float* col_mul,
                  int col_mul_stride, const void* bias_bf16, const void* residual_bf16, int64_t ldr, void* out_bf16,
                  int64_t ldo);

/* xaxb_gemm_fp8 with the format of each operand stated (0 = e4m3, non-zero = e5m2): the tensor core's
 * f8f6f4 kind takes either format on either side.  Serves fp8_matmul(..., fp8_dtype=float8_e5m2)
 * (xax/nn/fp8.py:347-378). */
int xaxb_gemm_fp8_formats(xaxb_ctx* ctx, void* stream, const void* a_fp8, int64_t lda, int a_is_e5m2,
                          const void* b_fp8, int64_t ldb, int b_is_e5m2, int64_t M, int64_t N, int64_t K,
                          const float* row_mul, int row_mul_stride, const float* col_mul, int col_mul_stride,
                          const void* bias_bf16, const void* residual_bf16, int64_t ldr, void* out_bf16, int64_t ldo);

/* Same contract for bf16 operands (lda/ldb in elements): the un-quantised linear /
 * lm_head einsum of xax/arch/attention.py:59-67 (xax/arch/llm.py:213-219). */
int xaxb_gemm_bf16(xaxb_ctx* ctx, void* stream, const void* a_bf16, int64_t lda, const void* b_bf16, int64_t ldb,
                   int64_t M, int64_t N, int64_t K, const float* row_mul, int row_mul_stride, const float* col_mul,
                   int col_mul_stride, const void* bias_bf16, const void* residual_bf16, int64_t ldr, void* out_bf16,
                   int64_t ldo);

/*
 * lm_head + cross-entropy loss / accuracy without materialising the logits (xax/arch/llm.py:718-887,
 * chunked_cross_entropy_loss and chunked_cross_entropy_acc, forward only): logits = hidden @ weight^T in
 * float32 (bf16 operands, float32 accumulation -- the reference casts the hidden states to float32 and
 * multiplies by the bf16 head), loss[t] = logsumexp(logits[t]) - logits[t, targets[t]], pred[t] = arg-max
 * (first index on ties).  The GEMM's epilogue reduces every 256-column slice of a row to (max, sum of
 * exponentials, target logit, arg-max) in registers; a second kernel merges the slices and a third takes
 * the masked means in a fixed order.  hidden: bf16 [T, H] (row stride ldh elements), weight: bf16 [V, H]
 * (row stride ldw), targets: int32 [T], mask: one byte per position (non-zero = counted) or NULL for all.
 * workspace: xaxb_lm_head_cross_entropy_workspace_bytes(T, V) bytes, 16-byte aligned.  Outputs: row_loss
 * float32 [T], row_pred int32 [T], result float32 [3] = {mean loss over counted positions (0 if none),
 * fraction of counted positions with pred == target, number counted}.
 */
int64_t xaxb_lm_head_cross_entropy_workspace_bytes(int64_t T, int64_t V);
int xaxb_lm_head_cross_entropy(xaxb_ctx* ctx, void* stream, const void* hidden_bf16, int64_t ldh, const void* weight_bf16,
                               int64_t ldw, int64_t T, int64_t V, int64_t H, const int32_t* targets, const uint8_t* mask,
                               void* workspace, int64_t workspace_bytes, float* row_loss, int32_t* row_pred,
                               float* result);

/* Test hook: force the tile width (32/64/128/256; 512, 448, 384 = the CTA-pair kernel with 256 x 256,
 * 256 x 224, 256 x 192 tiles where M > 128 and N >= 256; 0 = automatic) and the split-K factor
 * (1/2/4/8, 0 = automatic; > 1 needs M <= 128) of the following xaxb_gemm_* calls in this
 * process, so that tests can drive every kernel variant on the same inputs.  No counterpart
 * in the reference. */
int xaxb_gemm_force_plan(int bn, int split);

/* Requests to L2 for operand b (the weights: constant while a model runs) that carry no data to the SM:
 * a GEMM launched with programmatic dependent launch asks for the first `blocks_before_wait` 128-byte K
 * blocks of each CTA's first tile before it waits for the previous kernel of the stream (default 4; 0 =
 * nothing ahead of the wait).  Operand a and everything else is touched only after the wait, so results
 * do not depend on the setting; b must not be written by the kernel that precedes the GEMM in its
 * stream.  Process-wide.  No counterpart in the reference. */
int xaxb_gemm_set_prefetch(int blocks_before_wait);

/* Plain CUDA-core GEMM with the same contract as xaxb_gemm_fp8 (one thread per output,
 * float32 accumulation in k order).  A second opinion for the tensor-core kernel in tests;
 * never used by the module layer. */
int xaxb_gemm_fp8_check(xaxb_ctx* ctx, void* stream, const void* a_e4m3, int64_t lda, const void* b_e4m3,
                        int64_t ldb, int64_t M, int64_t N, int64_t K, const float* row_mul, int row_mul_stride,
                        const float* col_mul, int col_mul_stride, const void* bias_bf16, const void* residual_bf16,
                        int64_t ldr, void* out_bf16, int64_t ldo);

/* ---- small bandwidth kernels on the path ------------------------------------------- */

/*
 * RMSNorm (xax/arch/attention.py:96-98) over the last dimension of x[rows, dim] bf16 with
 * a bf16 weight, every intermediate rounded to bf16 as the reference's bf16 ops do.
 * y_bf16 may be NULL.  If q_e4m3 is non-NULL the row is also quantised with per-token
 * current scaling (as xaxb_quantize_current with group_rows = 1) from the normalised
 * values, writing q, scale and inv_scale.  If group_amax is non-NULL, max|y| of each group
 * of `group_rows` rows is accumulated into group_amax[row / group_rows] with an atomic max
 * on the float bits (caller clears it), for a following per-sequence quantisation.
 */
int xaxb_rmsnorm(xaxb_ctx* ctx, void* stream, const void* x_bf16, const void* weight_bf16, float eps, int64_t rows,
                 int64_t dim, void* y_bf16, void* q_e4m3, float* scale, float* inv_scale, float* group_amax,
                 int64_t group_rows);

/*
 * h = bf16(silu(gate) * up) with silu = bf16(g * bf16(sigmoid(g))) (xax/arch/attention.py:146).
 * gate and up are column blocks of one [rows, ld] bf16 buffer (the fused gate|up GEMM
 * output): gate = gu[:, 0:dim], up = gu[:, dim:2*dim] when up_bf16 is NULL, else separate
 * buffers with the same ld.  Quantisation outputs as in xaxb_rmsnorm.
 */
int xaxb_silu_mul(xaxb_ctx* ctx, void* stream, const void* gate_bf16, const void* up_bf16, int64_t ld, int64_t rows,
                  int64_t dim, void* h_bf16, void* q_e4m3, float* scale, float* inv_scale, float* group_amax,
                  int64_t group_rows);

/* amax[g] = max|x| over group g of `group_rows` rows (float32; cleared by the call): the first
 * pass of xaxb_quantize_current on its own, for tensor-parallel ranks that must max-reduce the
 * amax of a row-parallel layer's input across ranks before casting. */
int xaxb_group_amax(xaxb_ctx* ctx, void* stream, const void* x_bf16, int64_t rows, int64_t cols, int64_t group_rows,
                    float* amax);

/* Second pass of a per-group quantisation whose amax was accumulated by xaxb_rmsnorm /
 * xaxb_silu_mul: scales from group_amax, then the cast (same outputs as
 * xaxb_quantize_current; group_amax is read, not cleared). */
int xaxb_quantize_with_amax(xaxb_ctx* ctx, void* stream, const void* x_bf16, int64_t rows, int64_t cols,
                            int64_t group_rows, const float* group_amax, void* q_e4m3, float* scale,
                            float* inv_scale);

/* x[i, :] = table[tokens[i], :] (xax/arch/llm.py:205-207); bf16 rows of `dim` elements. */
int xaxb_embed(xaxb_ctx* ctx, void* stream, const int32_t* tokens, int64_t n_tokens, const void* table_bf16,
               int64_t vocab, int64_t dim, void* x_bf16);

/* out[i] = argmax_j float32(logits[i, j]), first index on ties, NaN counted as the maximum
 * (xax/arch/llm.py:1466-1470).  max_out (may be NULL) receives the winning value. */
int xaxb_argmax(xaxb_ctx* ctx, void* stream, const void* logits_bf16, int64_t rows, int64_t vocab, int64_t ld,
                int32_t* out, float* max_out);

/* Arg-max over a vocabulary split into `parts` slices of `slice` columns (the column-parallel
 * lm_head of xax/arch/llm.py:970-972): part_max / part_idx are [parts, rows] results of
 * xaxb_argmax on each slice; out[i] is the global index, lower index on ties. */
int xaxb_argmax_merge(xaxb_ctx* ctx, void* stream, const float* part_max, const int32_t* part_idx, int64_t parts,
                      int64_t rows, int64_t slice, int32_t* out);

/*
 * One token per row from logits [rows, vocab] bf16 (row stride ld) the way the generation loop picks it
 * (xax/arch/llm.py:1446-1489 with the masks of :1547-1570):
 *   - tokens outside [allowed_min, allowed_max) are masked (allowed_min < 0: no range); eos_id (< 0:
 *     none) is masked while allow_eos == 0 and, with a range, allowed in addition to it once
 *     allow_eos != 0; a masked logit counts as the most negative finite bf16;
 *   - temperature <= 0: arg-max in float32, first index on ties;
 *   - otherwise the logits are divided by the temperature, the nucleus is the tokens whose cumulative
 *     softmax probability in descending order (ties in index order) does not exceed top_p, the first
 *     always included, and out[r] is the token at quantile uniforms[r] (float32 in [0, 1), one per
 *     row) of the nucleus in that order.
 * The reference draws with jax.random.categorical from its own PRNG stream; the distribution is the
 * same, the random numbers are the caller's.  No sort: bisection on the 16-bit order of bf16 values.
 */
int xaxb_sample_top_p(xaxb_ctx* ctx, void* stream, const void* logits_bf16, int64_t rows, int64_t vocab, int64_t ld,
                      float temperature, float top_p, const float* uniforms, int32_t allowed_min,
                      int32_t allowed_max, int32_t eos_id, int allow_eos, int32_t* out);

/* ---- kernel 3: GQA attention with RoPE and a bf16 KV cache -------------------------- */

/*
 * RoPE + cache write for T new tokens of each of B sequences
 * (xax/arch/attention.py:870-888, rotation :510-515 "concatenated" style, every product
 * and sum rounded to bf16).  qkv: bf16 [B*T, ld] holding q | k | v column blocks
 * (Hq*D, Hkv*D, Hkv*D wide) -- the fused projection's output.  positions[b] = number of
 * tokens already cached for sequence b (the reference's cache["position"]).  cos/sin:
 * bf16 [table_len, D/2], built on the host in the reference's op order
 * (xax/arch/attention.py:390-397).
 * Writes q_rot [B*T, Hq, D] (rotated), k_cache/v_cache [B, max_len, Hkv, D] at rows
 * positions[b] .. positions[b]+T-1.  store_rotated_k = 1 keeps the reference's cache
 * contents (post-RoPE K); 0 stores K un-rotated for the rotate-on-load attention variant.
 * Returns XAXB_CACHE_OVERFLOW through the device status word if positions[b] + T > max_len.
 */
int xaxb_kv_append_rope(xaxb_ctx* ctx, void* stream, const void* qkv_bf16, int64_t ld, int64_t B, int64_t T,
                        int64_t Hq, int64_t Hkv, int64_t D, const int32_t* positions, const void* cos_bf16,
                        const void* sin_bf16, int64_t table_len, void* q_rot_bf16, void* k_cache_bf16,
                        void* v_cache_bf16, int64_t max_len, int store_rotated_k);

/* Bytes of float32 scratch xaxb_attn_decode needs for (B, Hq, D, max_len). */
int64_t xaxb_attn_decode_workspace_bytes(int64_t B, int64_t Hq, int64_t D, int64_t max_len);

/*
 * Decode attention: one query token per sequence against the cache
 * (xax/arch/attention.py:910-946 with seq_len = 1; softmax in float32; query head h reads
 * kv head h / (Hq/Hkv)).  q_rot: bf16 [B, Hq, D] already rotated; the query of sequence b
 * sits at positions[b] and attends to cache rows 0 .. positions[b] (the row written by the
 * preceding xaxb_kv_append_rope included).  k_is_rotated = 0 rotates K on load with the
 * cos/sin table (cos/sin may be NULL otherwise).  out: bf16 [B, Hq, D].
 * Split over 128-token chunks; per-chunk partial results go through `workspace`
 * (xaxb_attn_decode_workspace_bytes; contents need no initialisation).
 * A position outside 0 .. max_len - 1 is clamped into that range and reported as
 * XAXB_CACHE_OVERFLOW (site 15) through the device status word; the output stays finite.
 */
int xaxb_attn_decode(xaxb_ctx* ctx, void* stream, const void* q_rot_bf16, const void* k_cache_bf16,
                     const void* v_cache_bf16, const int32_t* positions, int64_t B, int64_t Hq, int64_t Hkv,
                     int64_t D, int64_t max_len, float softmax_scale, int k_is_rotated, const void* cos_bf16,
                     const void* sin_bf16, int64_t table_len, void* out_bf16, void* workspace,
                     int64_t workspace_bytes);

/* xaxb_attn_decode for a layer with a sliding window (xax/arch/attention.py:931-936: a query at
 * position q attends to keys q - window .. q; local_window_size of the block): chunks below the
 * window are never read.  K is expected rotated.  window < 0 means unlimited. */
int xaxb_attn_decode_window(xaxb_ctx* ctx, void* stream, const void* q_rot_bf16, const void* k_cache_bf16,
                            const void* v_cache_bf16, const int32_t* positions, int64_t B, int64_t Hq, int64_t Hkv,
                            int64_t D, int64_t max_len, float softmax_scale, int64_t window, void* out_bf16,
                            void* workspace, int64_t workspace_bytes);

/* Test hook: how many 128-token chunks one CTA of the decode-attention kernel walks.  0 or 1 = the
 * library's own choice (about four, fewer when that would leave SMs idle), 10 + n (n = 1 .. 64) = n.
 * Process-wide.  No counterpart in the reference. */
int xaxb_attn_decode_force_variant(int variant);

/*
 * xaxb_attn_decode with the per-token current-scaling cast of its output fused into the merge
 * pass: the row [Hq * D] of each sequence -- what the output projection consumes under the
 * vmapped Fp8Linear of xax/arch/attention.py:279 and :959-961 -- is written as e4m3 bytes with
 * row_scale / row_inv_scale (float32 [B]), bit-identical to xaxb_quantize_current(group_rows = 1)
 * applied to the bf16 output.  out_bf16 may be NULL.  Needs Hq <= 64 and Hq * D <= 4096.
 */
int xaxb_attn_decode_cast(xaxb_ctx* ctx, void* stream, const void* q_rot_bf16, const void* k_cache_bf16,
                          const void* v_cache_bf16, const int32_t* positions, int64_t B, int64_t Hq, int64_t Hkv,
                          int64_t D, int64_t max_len, float softmax_scale, int k_is_rotated, const void* cos_bf16,
                          const void* sin_bf16, int64_t table_len, void* out_bf16, void* q_e4m3, float* row_scale,
                          float* row_inv_scale, void* workspace, int64_t workspace_bytes);

/*
 * Decode attention without any memory from the caller beyond inputs and outputs.
 * No counterpart in the reference: this entry exists for callers that cannot allocate --
 * custom-call handlers that only see pre-declared buffers, serving loops that ban cudaMalloc
 * because it synchronises the device, embedders that keep the allocator to themselves.
 * Same contract and results as xaxb_attn_decode, but the per-chunk partial results go into
 * a 16 MiB array built into the library image (held by every GPU that loads the library until
 * the process exits; xaxb_attn_decode_static_capacity_bytes).  Shapes whose scratch
 * (xaxb_attn_decode_workspace_bytes) exceeds that are refused with XAXB_WORKSPACE_TOO_SMALL.
 * The context's device must be current.  The first call on a device looks up the array's
 * device address; make that first call outside any stream capture.  All calls share the
 * array: calls that overlap on the GPU race and must be serialised by the caller.
 */
int64_t xaxb_attn_decode_static_capacity_bytes(void);
int xaxb_attn_decode_static(xaxb_ctx* ctx, void* stream, const void* q_rot_bf16, const void* k_cache_bf16,
                            const void* v_cache_bf16, const int32_t* positions, int64_t B, int64_t Hq, int64_t Hkv,
                            int64_t D, int64_t max_len, float softmax_scale, int k_is_rotated, const void* cos_bf16,
                            const void* sin_bf16, int64_t table_len, void* out_bf16);

/*
 * Decode attention with the cache append fused in: xaxb_kv_append_rope (T = 1) + xaxb_attn_decode[_cast,
 * _window, _cast_tp] as one call, without the separate append launch and without the rotated-query
 * buffer.  qkv: bf16 [B, ld], the fused projection's output of the step's new token (q | k | v column
 * blocks as for xaxb_kv_append_rope), not yet in the cache; positions[b] = tokens already cached.  The
 * attention kernel rotates the query heads as it stages them, and the CTA that owns the cache chunk of
 * position positions[b] rotates the new key (k_is_rotated = 1; 0 stores and rotates on load as in
 * xaxb_attn_decode), places key and value into its tiles and writes them to cache row positions[b]:
 * results and cache contents are bit-identical to the two separate calls.  cos/sin [table_len >= max_len,
 * D/2] are always needed.  window < 0: unlimited.  out_bf16 and / or (q_e4m3, row_scale, row_inv_scale)
 * as in xaxb_attn_decode_cast; peer_bases != NULL with world > 1 adds the exchange of
 * xaxb_attn_decode_cast_tp.  positions are not advanced (xaxb_advance_positions).
 * (xax/arch/attention.py:870-946 for seq_len = 1.)
 */
int xaxb_attn_decode_append(xaxb_ctx* ctx, void* stream, const void* qkv_bf16, int64_t ld, void* k_cache_bf16,
                            void* v_cache_bf16, const int32_t* positions, int64_t B, int64_t Hq, int64_t Hkv,
                            int64_t D, int64_t max_len, float softmax_scale, int k_is_rotated, const void* cos_bf16,
                            const void* sin_bf16, int64_t table_len, int64_t window, void* out_bf16, void* q_e4m3,
                            float* row_scale, float* row_inv_scale, void* workspace, int64_t workspace_bytes,
                            void* const* peer_bases, int rank, int world, int64_t inbox_offset_bytes,
                            int64_t sync_offset_bytes);

/*
 * Causal prefill attention for T new tokens per sequence against the cache (which
 * already holds them, written by xaxb_kv_append_rope): query i of sequence b sits at
 * position positions[b] + i and attends to cache rows 0 .. positions[b] + i
 * (xax/arch/attention.py:914-926).  q_rot: bf16 [B*T, Hq, D]; out: bf16 [B*T, Hq, D].
 */
int xaxb_attn_prefill(xaxb_ctx* ctx, void* stream, const void* q_rot_bf16, const void* k_cache_bf16,
                      const void* v_cache_bf16, const int32_t* positions, int64_t B, int64_t T, int64_t Hq,
                      int64_t Hkv, int64_t D, int64_t max_len, float softmax_scale, void* out_bf16);

/* xaxb_attn_prefill with a sliding window (same rule as xaxb_attn_decode_window; KV tiles below
 * the first query's window are skipped). */
int xaxb_attn_prefill_window(xaxb_ctx* ctx, void* stream, const void* q_rot_bf16, const void* k_cache_bf16,
                             const void* v_cache_bf16, const int32_t* positions, int64_t B, int64_t T, int64_t Hq,
                             int64_t Hkv, int64_t D, int64_t max_len, float softmax_scale, int64_t window,
                             void* out_bf16);

/*
 * Cross-attention core (xax/arch/attention.py:1176-1182: jax.nn.dot_product_attention with
 * is_causal=False): T query rows per sequence, every one of which sees all kv_lens[b] rows of that
 * sequence's keys / values.  q: bf16 [B*T, Hq, D] (rotated by the caller where the block has RoPE);
 * k, v: bf16 [B, max_len, Hkv, D], rows kv_lens[b] .. max_len-1 ignored; query head h reads kv head
 * h / (Hq/Hkv).  The prefill kernel with its causal mask switched off.  out: bf16 [B*T, Hq, D].
 */
int xaxb_attn_cross(xaxb_ctx* ctx, void* stream, const void* q_bf16, const void* k_bf16, const void* v_bf16,
                    const int32_t* kv_lens, int64_t B, int64_t T, int64_t Hq, int64_t Hkv, int64_t D, int64_t max_len,
                    float softmax_scale, void* out_bf16);

/* Straightforward CUDA-core attention with the contract of xaxb_attn_prefill (T = 1 gives
 * decode): a second opinion for the tensor-core kernels in tests; never used by the
 * module layer. */
int xaxb_attn_check(xaxb_ctx* ctx, void* stream, const void* q_rot_bf16, const void* k_cache_bf16,
                    const void* v_cache_bf16, const int32_t* positions, int64_t B, int64_t T, int64_t Hq, int64_t Hkv,
                    int64_t D, int64_t max_len, float softmax_scale, void* out_bf16);

/* QK-norm (xax/arch/attention.py:864-867, the Qwen3 family): RMSNorm over head_dim of every query
 * and key head, in place on the fused projection output qkv [rows, (Hq + 2 Hkv) * D] (row stride
 * ld elements), to be called before xaxb_kv_append_rope.  Weights bf16 [D]; either may be NULL to
 * leave that side alone. */
int xaxb_qk_norm(xaxb_ctx* ctx, void* stream, void* qkv_bf16, int64_t ld, int64_t rows, int64_t Hq, int64_t Hkv,
                 int64_t D, const void* q_weight_bf16, const void* k_weight_bf16, float eps);

/* Rotary embedding on its own (RotaryEmbedding.apply_rotary_embeddings / _apply_rotary_4d,
 * xax/arch/attention.py:443-526): x and out bf16 [rows, heads, D], row r rotated with row
 * positions[r] of the cos / sin tables (bf16 [table_len, D/2]); interleaved = 0 is the
 * "concatenated" (LLaMA) style, 1 the "interleaved" (GPT-NeoX) style.  bf16 arithmetic in the
 * reference's op order; a position outside the table sets XAXB_CACHE_OVERFLOW. */
int xaxb_rope_apply(xaxb_ctx* ctx, void* stream, const void* x_bf16, int64_t rows, int64_t heads, int64_t D,
                    const int32_t* positions, const void* cos_bf16, const void* sin_bf16, int64_t table_len,
                    int interleaved, void* out_bf16);

/* positions[b] += delta for b < B (the reference's new_position = p + seq_len,
 * xax/arch/attention.py:888), kept on the device so a captured decode step can replay. */
int xaxb_advance_positions(xaxb_ctx* ctx, void* stream, int32_t* positions, int64_t B, int32_t delta);

/* ---- tensor-parallel exchange over NVLink peer memory ------------------------------- */

/*
 * The reference leaves tensor parallelism to XLA/GSPMD: xax/arch/llm.py:931-975 only names the
 * placement (o_proj and down are split along `in`), and the compiler inserts an all-reduce after
 * every row-parallel matmul.  These two entry points are that all-reduce for the decode step, on
 * buffers the caller has made visible to every GPU of the box ("symmetric" buffers: same size and
 * layout on every rank; peer_bases[r] is THIS process's mapping of rank r's buffer, a host array
 * of `world` device pointers, world <= 8).  The library allocates and maps nothing.
 *
 * Each exchange kind owns a flag region of xaxb_tp_sync_bytes() bytes inside the symmetric buffer
 * (sync_offset_bytes; zero-filled once, before the first call, on every rank).  Every rank must
 * issue the same sequence of calls.  One rank per GPU: these kernels wait for the matching kernel
 * on the other GPUs (bounded: XAXB_DEVICE_TIMEOUT in the status word when a peer never shows up).
 */
int64_t xaxb_tp_sync_bytes(void);
int64_t xaxb_tp_max_inbox_bytes(void);

/* out[rows, cols] (bf16, local) = sum over ranks of the bf16 partial outputs that every rank has
 * written at data_offset_bytes of its symmetric buffer; float32 accumulation in rank order, so
 * all ranks get the same bits.  rows <= 1024, cols % 8 == 0.  The caller alternates between two
 * data offsets from one call to the next (a buffer is free again two exchanges later). */
int xaxb_tp_allreduce_sum_bf16(xaxb_ctx* ctx, void* stream, void* const* peer_bases, int rank, int world,
                               int64_t data_offset_bytes, int64_t sync_offset_bytes, int64_t rows, int64_t cols,
                               void* out_bf16);

/* xaxb_tp_allreduce_sum_bf16 with the RMSNorm (xax/arch/attention.py:72-98) and the per-token
 * current-scaling e4m3 cast of the next FP8 projection applied to each summed row while it is in
 * registers: x_bf16 [rows, cols] receives the sum (the residual stream), q_e4m3 [rows, cols] and
 * row_scale / row_inv_scale [rows] what xaxb_rmsnorm(x, weight, eps) with a fused cast would have
 * produced from it, bit for bit.  cols <= 8192. */
int xaxb_tp_allreduce_sum_rmsnorm(xaxb_ctx* ctx, void* stream, void* const* peer_bases, int rank, int world,
                                  int64_t data_offset_bytes, int64_t sync_offset_bytes, int64_t rows, int64_t cols,
                                  void* x_bf16, const void* weight_bf16, float eps, void* q_e4m3, float* row_scale,
                                  float* row_inv_scale);

/*
 * The all-reduce fused into the row-parallel GEMM's epilogue (what xax/arch/llm.py:965-968 leaves to the
 * compiler after o_proj / down_proj), for the decode step (M <= 128 token rows).
 *
 * xaxb_gemm_fp8_push: xaxb_gemm_fp8 whose epilogue writes every 16-byte piece of the bf16 output straight
 *   into slot `rank` of EVERY rank's staging buffer (row-major [M, N] at slot_offset_bytes of each mapping in
 *   peer_bases; plain peer stores over NVLink) and then adds the number of pieces it completed to the 32-bit
 *   arrival counter at flag_offset_bytes of every rank's buffer (system-scope release).  No local `out`.
 * xaxb_tp_push_sum_rmsnorm: the consumer, one CTA per token row.  `staging` is THIS rank's buffer of `world`
 *   slots, slot_stride_bytes apart, `counter` its arrival counter, `totals` xaxb_tp_push_totals_bytes() of
 *   local memory, zero-filled once, holding the running number of pieces expected per row.  It waits (bounded,
 *   site 46) until world * rows * cols / 8 further pieces have arrived, sums the slots in rank order in
 *   float32 -- every rank gets the same bits -- and writes x_bf16 [rows, cols]; with weight_bf16 non-NULL also
 *   RMSNorm + per-token e4m3 cast of the sum as xaxb_tp_allreduce_sum_rmsnorm does.  It reads local memory only.
 * Staging buffer and counter must alternate between two pairs from one exchange to the next, every rank must
 * issue the same sequence, and a (staging, counter, totals) triple must see the same world on every use.
 */
int xaxb_gemm_fp8_push(xaxb_ctx* ctx, void* stream, const void* a_e4m3, int64_t lda, const void* b_e4m3, int64_t ldb,
                       int64_t M, int64_t N, int64_t K, const float* row_mul, int row_mul_stride, const float* col_mul,
                       int col_mul_stride, const void* bias_bf16, const void* residual_bf16, int64_t ldr,
                       void* const* peer_bases, int rank, int world, int64_t slot_offset_bytes,
                       int64_t flag_offset_bytes);
int64_t xaxb_tp_push_totals_bytes(void);
int xaxb_tp_push_sum_rmsnorm(xaxb_ctx* ctx, void* stream, const void* staging, int64_t slot_stride_bytes,
                             const void* counter, void* totals, int world, int64_t rows, int64_t cols, void* x_bf16,
                             const void* weight_bf16, float eps, void* q_e4m3, float* row_scale,
                             float* row_inv_scale);

/* The two places of a block where an activation amax spans the ranks, with the exchange done
 * inside the kernel that produces the activation (each CTA owns one token row: it pushes the
 * row's local amax to every rank, waits for theirs and casts with the maximum):
 *
 * xaxb_silu_mul_cast_tp: xaxb_silu_mul with the per-row e4m3 cast, the row being this rank's slice
 *   of the SwiGLU hidden activation that feeds the row-parallel down projection
 *   (xax/arch/attention.py:141-147 under the placement of xax/arch/llm.py:931-975).
 * xaxb_attn_decode_cast_tp: xaxb_attn_decode_cast (e4m3 output only) for this rank's query heads,
 *   feeding the row-parallel output projection (xax/arch/attention.py:959-961).
 *
 * rows / B <= 1024.  inbox_offset_bytes points at xaxb_tp_max_inbox_bytes() bytes and
 * sync_offset_bytes at xaxb_tp_sync_bytes() bytes of the symmetric buffer, both private to the
 * call site's exchange kind. */
int xaxb_silu_mul_cast_tp(xaxb_ctx* ctx, void* stream, const void* gate_bf16, const void* up_bf16, int64_t ld,
                          int64_t rows, int64_t dim, void* q_e4m3, float* scale, float* inv_scale,
                          void* const* peer_bases, int rank, int world, int64_t inbox_offset_bytes,
                          int64_t sync_offset_bytes);
int xaxb_attn_decode_cast_tp(xaxb_ctx* ctx, void* stream, const void* q_rot_bf16, const void* k_cache_bf16,
                             const void* v_cache_bf16, const int32_t* positions, int64_t B, int64_t Hq, int64_t Hkv,
                             int64_t D, int64_t max_len, float softmax_scale, int k_is_rotated, const void* cos_bf16,
                             const void* sin_bf16, int64_t table_len, void* q_e4m3, float* row_scale,
                             float* row_inv_scale, void* workspace, int64_t workspace_bytes, void* const* peer_bases,
                             int rank, int world, int64_t inbox_offset_bytes, int64_t sync_offset_bytes);

/* out[i] = max over ranks of in[i] for i < n <= 1024 (non-negative float32: the per-token amax
 * feeding a row-parallel FP8 projection; NaN wins, as in the quantiser).  inbox_offset_bytes
 * points at xaxb_tp_max_inbox_bytes() bytes of the symmetric buffer. */
int xaxb_tp_allreduce_max_f32(xaxb_ctx* ctx, void* stream, void* const* peer_bases, int rank, int world,
                              int64_t inbox_offset_bytes, int64_t sync_offset_bytes, const float* in, float* out,
                              int64_t n);

/* out[i] = arg-max over the whole vocabulary from per-rank slices: part_max / part_idx [rows] are
 * this rank's xaxb_argmax results on its `slice` columns (rank r holds columns r*slice ..), exchanged
 * through the symmetric buffer; every rank gets the same out (xax/arch/llm.py:970-972 shards the
 * lm_head along the vocabulary, :1466-1470 is the arg-max).  rows <= 1024; inbox_offset_bytes
 * points at xaxb_tp_argmax_inbox_bytes() bytes. */
int64_t xaxb_tp_argmax_inbox_bytes(void);
int xaxb_tp_argmax(xaxb_ctx* ctx, void* stream, void* const* peer_bases, int rank, int world,
                   int64_t inbox_offset_bytes, int64_t sync_offset_bytes, const float* part_max,
                   const int32_t* part_idx, int64_t rows, int64_t slice, int32_t* out);

#ifdef __cplusplus
}
#endif

#endif /* XAXB200_H_ */
