/*
 * fluxbin_b200 -- C ABI of the B200 (sm_100a) batch-1 packed-Linear decode kernels.
 *
 * This is the drop-in boundary: plain pointers and sizes, no framework types.  Every
 * entry point launches on the given CUDA stream, never synchronises and never throws;
 * unless its comment says otherwise it also never allocates.  Return value: 0 on
 * success, a negative FB_E* code on rejection (nothing was launched);
 * fb_last_error() then holds a message for the calling thread.
 * Device pointers must belong to the device that is current when the call is made.
 *
 * Citations name the reference project's interface each entry point replaces
 * (paths relative to the reference project's root).
 */
#ifndef FLUXBIN_B200_H_
#define FLUXBIN_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* 16-bit floating formats of activations, outputs and scales. */
#define FB_F16 0
#define FB_BF16 1

/* Error codes. */
#define FB_OK 0
#define FB_EINVAL (-1)  /* bad argument: null pointer, shape, dtype tag, alignment */
#define FB_ELIMIT (-2)  /* dimension outside the supported bounds */
#define FB_ESCRATCH (-3) /* scratch buffer missing or too small */
#define FB_ECUDA (-4)   /* a CUDA runtime call failed (message holds its text) */
#define FB_EALIAS (-5)  /* an output overlaps an input */

/* fb_w3_gemv flags. */
#define FB_W3_DECODED_BF16 1u /* add the +/-3 weight-rounding correction: the result then
                                 follows the dequantised 16-bit weight rather than
                                 scale * integer-dot (reference: "decoded_bf16" arithmetic,
                                 csrc/w3_lut.cu:105-122).  The dequantised weight is
                                 scale * (code - zero) rounded once in the scale's dtype.  Exact
                                 for zero points 3 and 4 (zeros == NULL is 4), where +/-3 are the
                                 only inexact products; other zero points get that correction
                                 only.  Zero points are then read before the lookups, which
                                 costs some speed. */

#define FB_W3_NO_PDL 2u /* launch without programmatic dependent launch (by default the
                          kernel's prologue may overlap the previous kernel in the stream;
                          it still waits for that kernel before reading x or writing) */
#define FB_W3_GROUP_PARTIALS 4u /* M = 1 only: `out` is an fp32 [G,O] workspace that receives
                                   each group's scaled sum instead of the reduced result
                                   (reference: inline_main, csrc/w3_lut.cu:251-273); follow
                                   with fb_w3_finish */

#define FB_W3_SAME_INPUT 8u /* the caller states that x (and perm) were complete before the launch DIRECTLY
                              ahead of this one in the stream began, that that launch is an fb_w3_gemv*
                              launch (these release their dependents only after their own wait) or an
                              ordinary launch, and that `out` and `scratch` are not touched by it: k_proj
                              behind q_proj, up_proj behind gate_proj on the same activations, each with
                              its own scratch.  The kernel then starts reading at once instead of waiting
                              for the launch ahead (about 1.3 us after that launch's last store) and
                              waits for it only before it ends, so stream order holds for whatever
                              follows.  At most three such launches in a row share no scratch if three
                              scratches rotate. */

typedef void* fb_stream_t; /* a cudaStream_t */

/* Message describing the last rejected call made by this thread ("" if none). */
const char* fb_last_error(void);

/* Library / device facts: key "version", "sm_count", "max_smem", "w3_max_m", "w3_mma_max_m",
 * "w3_max_splits", "w3_ctas_per_sm", "w3_smem_bytes", "tp_max_world".
 *  Returns the value, or FB_EINVAL for an unknown key. */
int64_t fb_query(const char* key);

/* Bytes of scratch fb_w3_gemv needs for a problem of this size (a status word, 2 MiB of
 * 64-bit combine words for the K split, and fp32 partials when K exceeds 4096).  The
 * scratch must be zero-filled once after allocation; every call leaves it ready for the next.  One scratch may be
 * shared by all calls that are ordered on one stream; calls that can overlap on the
 * GPU need separate scratch. */
size_t fb_w3_gemv_scratch_bytes(int m, int out_features, int in_features);

/*
 * y[M,O] = x[M,K] . W^T with W the GPTQ W3 group-128 planar layout:
 *   planes  uint8 [G,3,O,16]  bit planes of the codes, plane 2 stored inverted,
 *                             8 input positions per byte, LSB first (G = K/128)
 *   scales  f16|bf16 [G,O]
 *   zeros   uint8 [G,O] zero points, or NULL for the constant zero point 4
 *   perm    int16 [K] sorted position -> input column (desc_act), or NULL for identity
 * W[o, perm[k]] = scale[k/128, o] * (code - zero); accumulation in fp32.  The split over K
 * (up to 16 partial sums per output) is combined inside the kernel by 64-bit integer adds of
 * the partial sums in fixed point (steps of 2^-26), so results do not depend on arrival order:
 * repeat-exact and graph-replay-exact.  A partial sum that is not finite, or is 2^21 or more
 * in magnitude, has no fixed-point form: that output is written as NaN.
 * M = 1..4.  O % 32 == 0, G <= 255 (K <= 32640), O <= 65536; x, planes, scales, zeros 16-byte aligned.
 *
 * Replaces the reference's pybind entry points inline_main + finish and m1_out
 * (csrc/w3_lut.cu:251-332) and their launchers (:153-189).
 */
int fb_w3_gemv(const void* x, int act_dtype, int m, const uint8_t* planes, const void* scales,
               int scale_dtype, const uint8_t* zeros, const int16_t* perm, void* out,
               int out_features, int in_features, void* scratch, size_t scratch_bytes,
               unsigned flags, fb_stream_t stream);

/*
 * Several W3 matrices that share the activations x and K (q/k/v, or gate/up) in ONE launch:
 * the activation tables are built once per K block and the fixed cost of a launch is paid once.
 * Each matrix has its own planes / scales / zeros / out and out_features (a multiple of 32);
 * `residual` (optional, [M,O] in the activation dtype) is added to the rounded result, and the
 * sum is rounded again: out = T(T(y) + residual), what a Linear followed by an add produces.
 * Up to 4 matrices, at most 65536 rows in total; scratch sized for the total row count.
 * No counterpart in the reference, which launches every Linear on its own.
 */
typedef struct fb_w3_matrix {
  const uint8_t* planes;
  const void* scales;
  const uint8_t* zeros;   /* or NULL */
  void* out;
  const void* residual;   /* or NULL */
  int out_features;
} fb_w3_matrix_t;
int fb_w3_gemv_multi(const void* x, int act_dtype, int m, const fb_w3_matrix_t* matrices, int n_matrices,
                     int scale_dtype, const int16_t* perm, int in_features, void* scratch,
                     size_t scratch_bytes, unsigned flags, fb_stream_t stream);

/*
 * fb_w3_gemv_multi (M = 1, identity column order) with the producer of x fused into the table
 * build, which removes a launch from the decode step:
 *   FB_W3_INPUT_RMSNORM   x' = operand * T(x * rsqrt(mean(x^2) + eps)),  operand = norm weight [K]
 *   FB_W3_INPUT_SILU_MUL  x' = T(silu(x)) * operand,                     operand = the `up` vector [K]
 * with the roundings of the separate kernels (fb_rmsnorm, fb_silu_mul).  No counterpart in the
 * reference, where these are separate modules (fused_modules.py:30-63 and the stock MLP).
 */
#define FB_W3_INPUT_RMSNORM 1
#define FB_W3_INPUT_SILU_MUL 2
#define FB_W3_INPUT_ATTN_PIECES 3 /* fb_w3_gemv_push only: x = the pieces fb_attn_decode_partial left, eps = splits per head
                                     (what fb_w3_gemv_attn_merge does for the unsharded Linear) */
int fb_w3_gemv_fused_input(const void* x, int act_dtype, int transform, const void* operand, float eps,
                           const fb_w3_matrix_t* matrices, int n_matrices, int scale_dtype, int in_features,
                           void* scratch, size_t scratch_bytes, unsigned flags, fb_stream_t stream);

/*
 * The attention output as the fused input of the Linear that consumes it (o_proj): `partials` is
 * what fb_attn_decode_partial left, per head and split (output[128], max, sum) as fp32 at float
 * offset (16 * head + split) * 132; in_features = heads * 128.  The splits are merged while the
 * tables are built, with the arithmetic of fb_attn_decode's own last step (the results equal
 * fb_attn_decode_fused followed by fb_w3_gemv_multi bit for bit), which takes the cross-CTA merge
 * of the attention launch and its barrier off the critical path.  1..8 splits.
 */
int fb_w3_gemv_attn_merge(const void* partials, int splits, int act_dtype, const fb_w3_matrix_t* matrices,
                          int n_matrices, int scale_dtype, int in_features, void* scratch, size_t scratch_bytes,
                          unsigned flags, fb_stream_t stream);

/*
 * Tensor-parallel form of a row-split Linear (o_proj, down_proj): one matrix, M = 1, optional
 * fused input transform (0 = none) as in fb_w3_gemv_fused_input.  Instead of writing `out`
 * (ignored; may be any non-null pointer), the final fp32 value of output row o is stored,
 * together with a valid mark, as ONE 8-byte store {value, 1} to data[r][o] for every rank r
 * (pointers into each rank's exchange buffer of 8-byte slots, peer-mapped over NVLink, this
 * rank's own included).  fb_tp_reduce on each rank polls the slots and sums the ranks' rows:
 * compute and exchange are one kernel, the transfer overlaps the rest of the GEMV, there is no
 * fence, no counter and no collective library call between the two Linears.
 * No counterpart in the reference (single GPU only, engine_interface.py:26-27).
 */
typedef struct fb_w3_push {
  void* data[8];
  int world;
} fb_w3_push_t;
int fb_w3_gemv_push(const void* x, int act_dtype, int transform, const void* operand, float eps,
                    const fb_w3_matrix_t* matrix, int scale_dtype, int in_features, const fb_w3_push_t* push,
                    void* scratch, size_t scratch_bytes, unsigned flags, fb_stream_t stream);

/*
 * out[i] = T(T(sum_r value(parts[r*n + i])) + residual[i]) for i < n: the receiving half of
 * fb_w3_gemv_push.  `parts` is this rank's exchange buffer, [world, n] 8-byte slots, all zero
 * before the first use; a thread waits until the slots of its element carry the mark, sums them
 * in ascending rank order and zeroes them again.  The wait is bounded by wait_ns nanoseconds
 * (0 = the default of ten seconds, at most 60 s); on expiry *status is set to 4, the sum is of
 * whatever arrived and the slots are zeroed all the same.  The host reads *status after
 * synchronising; a non-zero value means the outputs of that step are invalid.  residual may be NULL.
 */
int fb_tp_reduce(void* parts, int world, const void* residual, void* out, int n, int dtype, unsigned* status,
                 uint64_t wait_ns, fb_stream_t stream);

/*
 * Small-batch form on the tensor cores: y[M,O] = x[M,K] . W^T for M = 1..16, same layout and
 * dtypes as fb_w3_gemv.  Every weight is dequantised once, T((code - zero) * scale) with T the
 * activation dtype, into a shared-memory operand tile and applied to all M rows by tcgen05.mma
 * (fp32 accumulation in tensor memory), so the time does not grow with M.  The K split is
 * combined as in fb_w3_gemv (repeat-exact).  Own scratch (zero-filled once, 256-byte aligned),
 * not to be shared with the other kernels.  The reference has no packed path for M > 1
 * (csrc/w3_lut.cu:195); its dense fallback (w3_lut_deployment.py:343-359) is the oracle.
 */
size_t fb_w3_gemm_small_scratch_bytes(int m, int out_features, int in_features);
int fb_w3_gemm_small(const void* x, int act_dtype, int m, const uint8_t* planes, const void* scales, int scale_dtype,
                     const uint8_t* zeros, const int16_t* perm, void* out, int out_features, int in_features,
                     void* scratch, size_t scratch_bytes, fb_stream_t stream);

/*
 * out[o] = T( sum_s partials[s, o] ), rows summed in ascending order.
 * partials fp32 [splits, O]; out f16|bf16 [O].
 * Replaces the reference's finish (csrc/w3_lut.cu:275-296, kernel :142-150).
 */
int fb_w3_finish(const float* partials, int splits, int out_features, void* out, int out_dtype,
                 fb_stream_t stream);

/*
 * Two-base binary-basis GEMV, M = 1, reference hybrid g128-s8 kernel layout (G = K/128):
 *   codes        uint8 [G,O,2,16] (planar != 0) or [G,O,32] (interleaved, planar == 0)
 *   rows         f32 [G,O,2]      cols         f32 [G,128,2]
 *   sparse_codes uint8 [G,O,2,1] (planar) or [G,O,2] (interleaved)
 *   sparse_rows  f32 [G,O,2]      sparse_cols  f32 [G,8,2]      indices int16 [G,8]
 * y[o] = sum_g ( r0*d0 + r1*d1 + sr0*s0 + sr1*s1 ), d_b = sum_k sign_b*col_b*x over the group,
 * s_b the same over the group's 8 refined columns; fp32 within a group; the groups (at most 255)
 * are combined by 64-bit fixed-point integer adds (steps of 2^-26, order-independent, so
 * repeat-exact; a group's term that is not finite or is 8192 or more in magnitude gives NaN).
 * Any O in 1..65536; scratch zero-filled once and 256-byte aligned, not shared with other
 * kernels, sized by fb_bb_gemv_scratch_bytes(O, K, 0).
 * Replaces the reference's m1_out of the v5 kernels (csrc/m1_v5.cu:132-195); all the
 * reference's kernel names map to this one entry point.
 */
size_t fb_bb_gemv_scratch_bytes(int out_features, int in_features, int global_scales);
int fb_bb_gemv(const void* x, int act_dtype, const uint8_t* codes, int planar, const float* rows,
               const float* cols, const uint8_t* sparse_codes, const float* sparse_rows,
               const float* sparse_cols, const int16_t* indices, void* out, int out_features,
               int in_features, void* scratch, size_t scratch_bytes, unsigned flags, fb_stream_t stream);

/*
 * Two-base GEMV with matrix-wide scales:  W = sum_b diag(r_b) B_b diag(c_b) + dense residual
 * columns.  codes uint8 [G,O,2,16] planar sign bits; row_scales f16 [2,O]; col_scales f16 [2,K];
 * salient_idx int32 [n] input columns; salient bf16 [O,n] added weights on those columns.
 * Scratch sized by fb_bb_gemv_scratch_bytes(O, K, 1).  The two-base part follows the
 * reference's global materialiser (evaluation.py:59-95) with one scale per row and per column.
 */
int fb_bb_global_gemv(const void* x, int act_dtype, const uint8_t* codes, const void* row_scales,
                      const void* col_scales, const int32_t* salient_idx, const void* salient,
                      int n_salient, void* out, int out_features, int in_features, void* scratch,
                      size_t scratch_bytes, unsigned flags, fb_stream_t stream);

/*
 * RMSNorm over `rows` vectors of `dim` 16-bit values:
 *   out = weight * T( x_f32 * rsqrt(mean(x_f32^2) + eps) )   (cast to T before the weight multiply)
 * x, out [rows, dim] contiguous; weight [dim]; out may alias x.
 * Replaces the reference's compiled RMSNorm forward (fused_modules.py:30-63).
 */
int fb_rmsnorm(const void* x, const void* weight, void* out, int rows, int dim, float eps, int dtype,
               fb_stream_t stream);

/*
 * Rotary embedding of one token's q heads [q_heads, head_dim] and k heads [k_heads, head_dim]
 * with one cos/sin row [head_dim]:  out = T( T(v*cos) + rotate_half(v)*sin ).
 * q_out / k_out may alias q / k.
 * Replaces the reference's fused_apply_rotary_pos_emb for a single position (fused_modules.py:66-85).
 */
int fb_rope_qk(const void* q, const void* k, const void* cosv, const void* sinv, void* q_out, void* k_out,
               int q_heads, int k_heads, int head_dim, int dtype, fb_stream_t stream);

/*
 * Glue kernels of one decode step.  The reference leaves these steps to stock HF modules
 * (static_decode.py:43-76: Qwen3 attention with q/k RMSNorm, rotary embedding, StaticCache update,
 * SDPA, and the SwiGLU MLP); they have no kernel of their own there.
 *
 * fb_qknorm_rope_cache: q [q_heads,D], k/v [kv_heads,D] of the new token -> per-head RMSNorm of q
 *   and k (weights [D]), rotary embedding with cos/sin [D], rotated q to q_out, rotated k and v
 *   into k_cache / v_cache [kv_heads, max_positions, D] at `position`.
 * fb_attn_decode: softmax(q k^T * scale) v over cache positions 0..length-1, grouped-query heads,
 *   D = 128; out [q_heads, D].  Positions are split over 1, 2, 4 or 8 CTAs per head, which form a
 *   thread-block cluster and merge their partial results through distributed shared memory;
 *   `scratch` (fb_attn_decode_scratch_bytes, zero-filled once, 16-byte aligned) is kept for the
 *   variant without clusters (partial results and one ticket per head).
 * fb_silu_mul: out[i] = T(silu(gate[i])) * up[i].
 */
int fb_qknorm_rope_cache(const void* q, const void* k, const void* v, const void* q_weight, const void* k_weight,
                         const void* cosv, const void* sinv, void* q_out, void* k_cache, void* v_cache, int q_heads,
                         int kv_heads, int head_dim, int position, int max_positions, float eps, int dtype,
                         fb_stream_t stream);
size_t fb_attn_decode_scratch_bytes(int q_heads);
int fb_attn_decode(const void* q, const void* k_cache, const void* v_cache, void* out, int q_heads, int kv_heads,
                   int head_dim, int length, int max_positions, float scale, int dtype, void* scratch,
                   size_t scratch_bytes, fb_stream_t stream);

/*
 * fb_qknorm_rope_cache and fb_attn_decode in ONE launch: q, k, v are the raw rows of the new
 * token; every CTA norms and rotates the q head it serves (and the new k) itself, uses the new
 * token's k / v directly and one CTA per k/v head writes them into cache row `position`.
 * Attends over positions 0..position.  Same results, bit for bit, as the two calls.
 * Ordering: the norm weights, the rotary row and the cache rows of positions < `position` are read
 * BEFORE the kernel waits for the launch ahead of it in the stream, so they must be complete when
 * that launch begins (weights and rotary tables are constants of a decode).  For the cache rows that holds
 * when they were written by ordinary (not programmatically dependent) work, or by an earlier
 * fb_attn_decode_fused with at least one fb_attn_decode_fused or fb_lm_head_argmax launch, or any
 * ordinary launch, between it and this call: those kernels release their dependents only after
 * their own wait.  A decode loop (one such call per layer and step, the LM head between steps)
 * satisfies this by construction; two calls on the same cache directly behind each other, or with
 * only fb_w3_gemv launches between them, do not.
 */
int fb_attn_decode_fused(const void* q, const void* k, const void* v, const void* q_weight, const void* k_weight,
                         const void* cosv, const void* sinv, void* k_cache, void* v_cache, void* out, int q_heads,
                         int kv_heads, int head_dim, int position, int max_positions, float eps, float scale, int dtype,
                         void* scratch, size_t scratch_bytes, fb_stream_t stream);

/*
 * fb_attn_decode_fused without its last step: every CTA leaves the (output, max, sum) of its share
 * of the positions in `partials` (fb_attn_decode_scratch_bytes(q_heads) bytes, 16-byte aligned; no
 * need to zero it) for fb_w3_gemv_attn_merge; fb_attn_decode_splits(position + 1) is the number of
 * splits per head it uses.  Same ordering rules as fb_attn_decode_fused.
 */
int fb_attn_decode_splits(int length);
int fb_attn_decode_partial(const void* q, const void* k, const void* v, const void* q_weight, const void* k_weight,
                           const void* cosv, const void* sinv, void* k_cache, void* v_cache, int q_heads, int kv_heads,
                           int head_dim, int position, int max_positions, float eps, float scale, int dtype,
                           void* partials, size_t partial_bytes, fb_stream_t stream);

int fb_silu_mul(const void* gate, const void* up, void* out, int n, int dtype, fb_stream_t stream);

/*
 * LM head of a greedy decode step in one launch:
 *   x' = norm_weight ? norm_weight * T(x * rsqrt(mean(x^2) + eps)) : x     (the final RMSNorm, as fb_rmsnorm)
 *   logit[v] = T( sum_k weight[v,k] * x'[k] )   fp32 accumulation, weight f16|bf16 [vocab, K] row-major
 *   *best = the lowest v whose logit is the largest (torch.argmax's tie rule on the 16-bit logits)
 * `logits` (optional, [vocab]) receives the 16-bit logits; without it they never leave the chip.
 * `embedding` + `next_hidden` (optional, together): after the choice is known, row
 * (*forced_next if forced_next else *best) of embedding [vocab, K] is copied to next_hidden [K], so that the
 * next step starts without a gather launch; next_hidden may be x itself (the copy happens after every
 * CTA has staged x).  scratch: fb_lm_head_scratch_bytes() bytes, 16-byte
 * aligned, zero-filled once; every call leaves it zero.  K a multiple of 8.
 * The reference keeps this step as the stock 16-bit Linear plus torch.argmax and names it the next
 * thing to fuse (docs/performance/NONLINEAR_FUSION.md:100); the embedding lookup is the stock module.
 */
size_t fb_lm_head_scratch_bytes(void);
int fb_lm_head_argmax(const void* x, const void* norm_weight, float eps, const void* weight, int vocab, int in_features,
                      int dtype, void* logits, int64_t* best, const int64_t* forced_next, const void* embedding,
                      void* next_hidden, void* scratch, size_t scratch_bytes, fb_stream_t stream);

/* out[0..K) = embedding[*token, 0..K): the embedding lookup of one token id held on the device. */
int fb_embed_row(const void* embedding, const int64_t* token, void* out, int vocab, int in_features, fb_stream_t stream);

/*
 * The LM head split by vocabulary rows over tensor-parallel ranks.  fb_lm_head_shard runs
 * fb_lm_head_argmax's kernel over rows row_base .. row_base + vocab_rows - 1 (`weight` points at
 * the shard's first row, `logits`, if given, at the shard's first logit) and, instead of
 * publishing a choice, stores the shard's best key (rounded logit and global row) into slot `rank`
 * of every rank's key array (`keys`: one array of `world` 8-byte words per rank, zero before first
 * use; peer pointers, plain stores, no multicast).  fb_tp_argmax, launched after it on every rank,
 * polls this rank's `world` slots (bounded: wait_ns as in fb_tp_reduce; status 6 on expiry), takes
 * the largest key (ties: the lowest row), zeroes the slots, writes the chosen row to `best` and,
 * when given, copies the embedding row of `forced_next` (or of the choice) into `next_hidden`.
 * Every rank thus holds the same choice without a collective call.  No counterpart in the reference.
 */
int fb_lm_head_shard(const void* x, const void* norm_weight, float eps, const void* weight, int vocab_rows, int row_base,
                     int in_features, int dtype, void* logits, const fb_w3_push_t* keys, int rank, void* scratch,
                     size_t scratch_bytes, fb_stream_t stream);
int fb_tp_argmax(void* keys, int world, int64_t* best, const int64_t* forced_next, const void* embedding, void* next_hidden,
                 int vocab, int in_features, unsigned* status, uint64_t wait_ns, fb_stream_t stream);

/*
 * fb_w3_gemv without a scratch argument, for callers that cannot allocate device memory where
 * they call this library (all memory already handed to a pool, a framework allocator that must
 * not be bypassed, a CUDA graph capture in progress).  The split-K scratch is a fixed array of
 * FB_W3_STATIC_SCRATCH_BYTES inside the library, resident on every GPU that loads it.
 * Same arguments and results as fb_w3_gemv; problems whose scratch need
 * (fb_w3_gemv_scratch_bytes) exceeds that size are rejected with FB_ELIMIT.  This call itself
 * allocates nothing.  The first call on a device looks up the array's device address; make that
 * first call before any stream capture.  All calls on a device share the one array: the control
 * block is cleared on the stream at every call, and two calls that can overlap on the GPU race.
 * The device-side status word (an expired bounded wait) lives in that control block too and is
 * wiped by the next call's clear, so it cannot be observed through this entry point: callers that
 * need it use fb_w3_gemv with their own scratch.
 * It has no counterpart in the reference, whose callers always pass a workspace.
 */
#define FB_W3_STATIC_SCRATCH_BYTES (4u << 20)
int fb_w3_gemv_static(const void* x, int act_dtype, int m, const uint8_t* planes, const void* scales,
                      int scale_dtype, const uint8_t* zeros, const int16_t* perm, void* out,
                      int out_features, int in_features, unsigned flags, fb_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* FLUXBIN_B200_H_ */
