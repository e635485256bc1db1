/*
 * atma_b200 - C ABI of the B200 (sm_100a) kernels for ATMA's global-mixing hot path.
 *
 * Every entry point takes plain device pointers, sizes, element strides and a CUDA
 * stream (passed as void*; NULL = the legacy default stream).  Nothing here allocates
 * or synchronises unless its comment says so; outputs and scratch are caller-owned.
 * All calls return ATMA_OK (0) or a negative atma_status; atma_last_error() returns a
 * message for the calling thread's last failure.
 *
 * Each declaration names the function of the reference (akbar2habibullah/atma) whose
 * device work it replaces, by path:line inside that project.
 */
#ifndef ATMA_B200_H_
#define ATMA_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum { ATMA_OK = 0, ATMA_ERR_INVALID = -1, ATMA_ERR_CUDA = -2, ATMA_ERR_UNSUPPORTED = -3 } atma_status;

/* Element types of activations / caches.  Statistics and recurrent state are always fp32. */
typedef enum { ATMA_F32 = 0, ATMA_BF16 = 1, ATMA_F16 = 2 } atma_dtype;

const char* atma_last_error(void);
int atma_abi_version(void);

/* ------------------------------------------------------------------------------------
 * Polar Attention prefill.
 * Replaces kernel/polar_triton.py:49-191 (_polar_fwd_kernel) as launched by
 * _polar_forward (:505-590) behind polar_attention_fwd (:594-609), and - with a tile map
 * - kernel/polar_triton.py:194-309 / :613-669 (polar_attention_packed_fwd).
 *
 * q is [B][H][Tq][dk], k and v are [B][Hkv][Tk][dk] addressed through element strides
 * (innermost dimension contiguous), so both (B,H,T,dk) and (B,T,H,dk) storage work and
 * K/V need NOT be expanded to H heads (Hkv must divide H; head h reads KV head
 * h / (H/Hkv)).  Key j (absolute position key_offset + j) is visible to query i iff
 * pos < n_i and (window > 0) pos >= n_i - window.  n_i comes from n_keys[i] (fp32,
 * length Tq) or, when n_keys is NULL, n_i = n_base + i + 1.
 *
 * spg, sps, beta are softplus(len_gain_raw), softplus(null_slope_raw),
 * softplus(mag_beta_raw) - the host applies softplus as polar_triton.py:540-542 does.
 *
 * Streaming statistics (all fp32): m, L, Q2 are [B][H][Tq], S is [B][H][Tq][dk], dense.
 * stats_in  != NULL: continue from the statistics of earlier key blocks (ring pass).
 * finalize  != 0   : fold the null sink and write c [B][H][Tq][dk] (strided, dtype) and
 *                    mag [B][H][Tq] (strided, dtype).
 * finalize  == 0   : write the running statistics to stats_out instead (c, mag unused).
 *
 * Packed mode (n_tiles > 0): B must be 1 and q, k, v are the packed [tokens][heads][dk]
 * arrays (pass their strides as h- and t-strides); tile t covers query rows
 * tile_q_start[t] .. +127 of the sequence that starts at packed row tile_seq_start[t]
 * and has tile_seq_len[t] tokens; n_i = local query index + 1.
 * ---------------------------------------------------------------------------------- */
typedef struct {
  const void* q; const void* k; const void* v;
  int64_t q_sb, q_sh, q_st;          /* element strides; innermost stride must be 1 */
  int64_t k_sb, k_sh, k_st;
  int64_t v_sb, v_sh, v_st;
  void* c; int64_t c_sb, c_sh, c_st;
  void* mag; int64_t mag_sb, mag_sh, mag_st;
  const float* n_keys;               /* [Tq] or NULL */
  float n_base;                      /* used when n_keys == NULL */
  int64_t key_offset;                /* absolute position of key row 0 */
  const float* v_null;               /* [H][dk] fp32 */
  const float* spg; const float* null_base; const float* sps; const float* beta;  /* [H] fp32 */
  const float* stats_in_m; const float* stats_in_l; const float* stats_in_q2; const float* stats_in_s;
  float* stats_out_m; float* stats_out_l; float* stats_out_q2; float* stats_out_s;
  int finalize;
  int B, H, Hkv, Tq, Tk, dk;
  int dtype;                         /* atma_dtype of q, k, v, c, mag */
  int window;                        /* 0 = full context */
  float eps;
  const int32_t* tile_seq_start; const int32_t* tile_q_start; const int32_t* tile_seq_len;
  int n_tiles;                       /* 0 = dense mode */
} atma_polar_prefill_args;

int atma_polar_prefill(const atma_polar_prefill_args* args, void* stream);

/* Which implementation atma_polar_prefill would run for these arguments:
 * 1 = tcgen05/TMEM/TMA tile kernel (16-bit, dk = 128), 0 = fp32 CUDA-core kernel. */
int atma_polar_prefill_path(const atma_polar_prefill_args* args);

/* Every wait inside the tensor-core kernels is bounded; a CTA whose wait ran out returns
 * early and sets a device status word.  This call synchronises the device, writes the word
 * (0 = no wait ever ran out) to *status and clears it.  (Diagnostic; no reference counterpart.) */
int atma_device_status(int* status);

/* ------------------------------------------------------------------------------------
 * Paged Polar decode.  Replaces kernel/polar_triton.py:681-792 (_polar_decode_kernel)
 * behind polar_attention_decode (:796-858).
 * q [B][H][dk] (dense); k_cache, v_cache [num_blocks][block_size][Hkv][dk] (dense);
 * block_tables int32 [B][max_blocks] (row stride bt_stride); context_lens int32 [B].
 * c [B][H][dk], mag [B][H] in `dtype`.
 * The context of each (sequence, KV head) is cut into n_splits key ranges that run as
 * separate CTAs; their partial statistics go through `scratch` (fp32, at least
 * atma_polar_decode_scratch_floats(B, H, dk, n_splits) floats) and a second kernel
 * merges them and folds the null sink.  Launch shapes depend only on the arguments
 * passed here, never on device data, so the call can be captured in a CUDA graph.
 * ---------------------------------------------------------------------------------- */
typedef struct {
  const void* q; const void* k_cache; const void* v_cache;
  const int32_t* block_tables; int64_t bt_stride;
  const int32_t* context_lens;
  const float* v_null; const float* spg; const float* null_base; const float* sps; const float* beta;
  void* c; void* mag;
  float* scratch;
  int B, H, Hkv, dk, block_size, max_blocks, num_blocks;
  int n_splits;
  int dtype;
  int window;
  float eps;
  /* Optional fused epilogue and output placement (all zero / NULL = plain dense c and mag).
   * gate [B][H][dk] with element strides (gate_sb, gate_sh): c is written as c * sigmoid(gate),
   * the operand of the output projection (inference/models/atma.py:246-252), with the roundings
   * of the separate eager ops.  c_sb / mag_sb: element stride between the rows of c and of mag
   * (0 = dense), so that both can land in one row of a wider activation buffer. */
  const void* gate; int64_t gate_sb, gate_sh;
  int64_t c_sb, mag_sb;
  /* A context whose keys are spread over several caches (a sequence prefilled context-parallel
   * over several GPUs): context_lens then counts the keys of THIS cache, temp_lens int32 [B] the
   * whole context, which sets the per-query temperature (NULL = context_lens); skip_merge != 0
   * stops after the key-range pass and leaves the partial statistics in `scratch`:
   * [B*H][n_splits]{m, L, Q2, 0} followed by [B*H][n_splits][dk] sums.  atma_polar_decode_merge
   * then merges any number of such partials (this cache's and the peers', laid out the same way
   * with n_splits = their total count) with context_lens = the whole context; it reads scratch,
   * context_lens, the five parameter arrays, B, H, dk, n_splits, window, dtype, eps and the output
   * fields.  Windowed attention is not available in this form. */
  const int32_t* temp_lens;
  int skip_merge;
  /* Optional: the K/V rows of the token being decoded, [B][Hkv][dk] with row strides in elements, and their
   * cache rows append_slots[B] (int32, negative = skip).  The key-range kernel then stores them itself before
   * it reads the cache (the CTA whose key range ends with the new token does it), which replaces the
   * store_kvcache launch that precedes the decode call (inference/layers/attention.py:30-56,85-97).  Honoured
   * for 16-bit caches with head_dim 64 or 128 and at most 8 query heads per KV head; callers check
   * atma_polar_decode_appends() and otherwise call atma_store_kvcache first. */
  const void* append_k; const void* append_v;
  int64_t append_k_stride, append_v_stride;
  const int32_t* append_slots;
} atma_polar_decode_args;

int64_t atma_polar_decode_scratch_floats(int B, int H, int dk, int n_splits);
int atma_polar_decode(const atma_polar_decode_args* args, void* stream);
int atma_polar_decode_merge(const atma_polar_decode_args* args, void* stream);
/* 1 if atma_polar_decode would store the append_* rows itself for this dtype / head_dim / head grouping, else 0. */
int atma_polar_decode_appends(const atma_polar_decode_args* args);

/* ------------------------------------------------------------------------------------
 * Paged Polar decode for callers that cannot allocate device memory.  (No counterpart in
 * the reference, whose Python wrapper allocates freely.)
 * Same arguments and results as atma_polar_decode, except that args->scratch is ignored:
 * the split partials go to an array built into the library image (4 MiB per GPU, held by
 * every GPU that loads the library until the process exits).  Meant for a host that has
 * given all free device memory to its KV cache, or that runs inside a fixed memory plan,
 * and so has no way to provide scratch at decode time.  The call makes no cudaMalloc,
 * cudaFree or other allocating call.
 *  - Limit: B*H*n_splits*(4+dk) must not exceed atma_polar_decode_static_max_floats()
 *    (1,048,576 floats; e.g. B=64, H=8, dk=128 allows n_splits <= 15).  Larger requests
 *    fail with ATMA_ERR_INVALID and a message; nothing is launched.
 *  - The first call on each device looks up the array's device address (with that device
 *    current); make that first call before any stream capture begins.
 *  - All calls on a device share the one array, which keeps the previous call's partials.
 *    Nothing in it has to start at zero: each call rewrites every entry it later reads.
 *    Two calls whose kernels overlap on the GPU (different streams) race on it - keep
 *    calls on one device ordered.
 * ---------------------------------------------------------------------------------- */
int64_t atma_polar_decode_static_max_floats(void);
int atma_polar_decode_static(const atma_polar_decode_args* args, void* stream);

/* ------------------------------------------------------------------------------------
 * Gated-delta decode step, in place on a slot-indexed state table.
 * Replaces kernel/gated_delta_triton.py:36-75 behind gated_delta_decode_step (:79-117).
 * q, k, v [B][H][d] with element strides (sb, sh), innermost contiguous, dtype `dtype`;
 * gamma, beta fp32 [B][H] dense; state fp32 [max_seqs][H][dk][dv] with strides
 * (state_ss, state_sh), [dk][dv] dense, UPDATED IN PLACE; slots int64 [B];
 * r fp32 [B][H][dv] dense.  A negative slot skips the row (its r is zeroed).
 * ---------------------------------------------------------------------------------- */
int atma_gated_delta_decode_step(const void* q, const void* k, const void* v,
                                 int64_t q_sb, int64_t q_sh, int64_t k_sb, int64_t k_sh,
                                 int64_t v_sb, int64_t v_sh, int dtype,
                                 const float* gamma, const float* beta,
                                 float* state, int64_t state_ss, int64_t state_sh,
                                 const int64_t* slots, float* r,
                                 int B, int H, int dk, int dv, float eps, void* stream);

/* The same step with the work around it folded in (16-bit or fp32 inputs, dk = dv = 128), one CTA per
 * (sequence, head) holding the whole 64 KiB state between its read and its write:
 *  - k, v carry Hkv un-expanded heads (head h reads KV head h / (H / Hkv)); the reference expands
 *    them first (inference/models/atma.py:609-611);
 *  - gamma / beta either as fp32 [B][H] (g_logit == NULL) or as the logits of the two gate
 *    projections in `dtype` with row stride logit_sb: gamma = sigmoid(g_logit + gamma_bias),
 *    beta = sigmoid(b_logit + beta_bias) (:352-355);
 *  - with gate != NULL the read-out is written as RMSNorm(r) * sigmoid(gate) in `dtype` to
 *    out [B][H*dv] (row strides gate_sb, out_sb), the operand of mem.proj (:373-375); else r goes
 *    out as fp32 [B][H][dv]. */
int atma_gated_delta_decode_step_fused(const void* q, const void* k, const void* v,
                                       int64_t q_sb, int64_t q_sh, int64_t k_sb, int64_t k_sh,
                                       int64_t v_sb, int64_t v_sh, int dtype, int Hkv,
                                       const float* gamma, const float* beta,
                                       const void* g_logit, const void* b_logit, int64_t logit_sb,
                                       float gamma_bias, float beta_bias,
                                       float* state, int64_t state_ss, int64_t state_sh,
                                       const int64_t* slots, float* r,
                                       const void* gate, int64_t gate_sb, void* out, int64_t out_sb,
                                       int B, int H, int dk, int dv, float eps, float rms_eps, void* stream);

/* ------------------------------------------------------------------------------------
 * Decode-side glue of a global layer in one launch (no single counterpart in the reference:
 * it is the run of ops at inference/models/atma.py:557-572 - F.rms_norm of q and k per head,
 * three _gpu_conv_step calls in residual form on the slot-indexed conv-state tables, and
 * store_kvcache of the new K/V row).  q_gate [B][H][2*dk] with element strides (qg_row, qg_head),
 * only the q half is read; k, v [B][Hkv][dk] with row strides; w_* [C][K]; state_* [rows][C][K-1]
 * with row strides ss_*, UPDATED IN PLACE at rows slots[b] (negative = padded batch row: the
 * conv sees a zero state and nothing is written); outputs dense; k_cache / v_cache rows
 * [slot][Hkv][dk] receive the post-conv K/V at slot_mapping[b] (-1 = skip), may be NULL.
 * ---------------------------------------------------------------------------------- */
int atma_qkv_prep_decode(const void* q_gate, int64_t qg_row, int64_t qg_head, const void* k, int64_t k_row,
                         const void* v, int64_t v_row, const void* w_q, const void* w_k, const void* w_v,
                         void* state_q, void* state_k, void* state_v, int64_t ss_q, int64_t ss_k, int64_t ss_v,
                         const int64_t* slots, void* q_out, void* k_out, void* v_out, void* k_cache,
                         void* v_cache, const int32_t* slot_mapping, int B, int H, int Hkv, int dk, int K,
                         float eps, int dtype, void* stream);

/* Residual add followed by the next RMSNorm: x_out = x + y (y may be NULL), h_out =
 * x_out * rsqrt(mean(x_out^2) + eps) * weight (weight may be NULL); rows of D <= 4096 values,
 * dense.  The block structure x + mix(norm1(x)), x + mlp(norm2(x)) of
 * inference/models/atma.py:709-712 (model/layers.py:14-17) is two of these per layer. */
int atma_add_rms_norm(const void* x, const void* y, const void* weight, void* x_out, void* h_out, int rows, int D,
                      float eps, int dtype, void* stream);

/* Weight-streaming linear layer for decode batches of up to 16 rows (16-bit types): out[b][n] =
 * sum_k x[b][k] * weight[n][k] + bias[n] (bias may be NULL), weight [N][K] dense in torch's Linear
 * layout, fp32 accumulation, one rounding to `dtype`.  gated != 0: the N outputs are the two halves
 * [first | second] of the MLP's fc projection and out[b][f] = second[f] * relu(first[f])^2 for f < N/2
 * (out has N/2 columns; bf16 rounds the square as eager execution does) - InferenceMLP.forward's
 * fc GEMM and squared_relu_gate in one launch (inference/models/atma.py:87-97); the plain form serves
 * its proj GEMM, the LFM2 in_proj / out_proj (:631-673) and the LM head at these batch sizes.
 * K a multiple of 32, N of 16 (32 when gated); x rows 16-byte aligned. */
int atma_decode_linear(const void* x, int64_t x_row_stride, const void* weight, const void* bias, void* out,
                       int64_t out_row_stride, int B, int N, int K, int gated, int dtype, void* stream);

/* ------------------------------------------------------------------------------------
 * Gated-delta chunked scan.  Replaces the third-party flash-linear-attention call
 * chunk_gated_delta_rule(q,k,v,g,beta,scale=1,initial_state,output_final_state,
 * use_qk_l2norm_in_kernel=True) made at inference/models/atma.py:285-287,318-322 and
 * model/blocks.py:48-49; semantics are those of model/blocks.py:375-423.
 * q [B][T][H][dk], k [B][T][Hkv][dk], v [B][T][Hkv][dv] dense, dtype `dtype` (Hkv divides H;
 * head h reads KV head h / (H/Hkv); the reference passes Hkv == H); g (log decay <= 0) and
 * beta fp32 [B][T][H]; initial_state fp32 [B][H][dk][dv] or NULL (zeros); o [B][T][H][dv] in
 * `dtype`; final_state fp32 [B][H][dk][dv] or NULL.  `scratch` holds the chunk-local
 * factors: at least atma_gated_delta_scan_scratch_bytes(B,T,H,dk,dv) bytes.
 * `normalize_qk` != 0 L2-normalises q and k rows in-kernel (x / max(||x||, 1e-12), as
 * F.normalize does); `scale` multiplies q.
 * ---------------------------------------------------------------------------------- */
int64_t atma_gated_delta_scan_scratch_bytes(int B, int T, int H, int dk, int dv);
int atma_gated_delta_scan(const void* q, const void* k, const void* v, int dtype,
                          const float* g, const float* beta,
                          const float* initial_state, void* o, float* final_state,
                          void* scratch, int B, int T, int H, int Hkv, int dk, int dv,
                          int normalize_qk, float scale, void* stream);
/* The same call with the cut of each sequence along T stated (16-bit inputs, dk = dv = 128;
 * ignored otherwise).  A batch of few sequences and heads leaves most SMs idle in the recurrence
 * over the chunks, so the sequence is cut into `segments` pieces that are walked side by side:
 * a first pass gives every later segment's affine map on the state (segment 0 runs for real), the
 * maps are chained into the state at the start of each segment, a second pass runs the later
 * segments from those states.  Results are those of the single pass within rounding (the same
 * hand-over the reference does between prefill chunks, inference/models/atma.py:509-544).
 * segments = 1: single pass (least total work - for a scan that runs beside other kernels);
 * 2..16: that many segments; 0: chosen from B, H and T (what atma_gated_delta_scan does). */
int atma_gated_delta_scan_segmented(const void* q, const void* k, const void* v, int dtype,
                                    const float* g, const float* beta,
                                    const float* initial_state, void* o, float* final_state,
                                    void* scratch, int B, int T, int H, int Hkv, int dk, int dv,
                                    int normalize_qk, float scale, int segments, void* stream);

/* ------------------------------------------------------------------------------------
 * The two halves of atma_gated_delta_scan, for a sequence that is split across GPUs.
 * (The reference has no multi-GPU path; its single-device statement of the same hand-over is
 * the chunked-prefill state carry of inference/models/atma.py:262-301.)
 * _factors builds the state-independent per-chunk factors of B sequences into `scratch`
 * (16-bit inputs, dk = dv = 128 only; arguments as atma_gated_delta_scan).
 * _recur runs n_rec (<= 64) recurrences over those factors: recurrence i uses the factors of
 * sequence rec_of[i] (host array, NULL = identity), starts from initial_state[i] (fp32
 * [n_rec][H][dk][dv], NULL = zeros), writes o[i] ([n_rec][T][H][dv], NULL = no outputs) and
 * final_state[i].  zero_u0[i] != 0 (host array, NULL = all 0) runs the recurrence with v = 0:
 * started from the identity it returns the matrix P of the segment's affine state map
 * S_out = P S_in + Q, while the plain recurrence started from zero returns Q.
 * ---------------------------------------------------------------------------------- */
int atma_gated_delta_scan_factors(const void* q, const void* k, const void* v, int dtype,
                                  const float* g, const float* beta, void* scratch,
                                  int B, int T, int H, int Hkv, int dk, int dv,
                                  int normalize_qk, float scale, void* stream);
int atma_gated_delta_scan_recur(void* scratch, int dtype, int B, int T, int H, int dk, int dv,
                                int n_rec, const int* rec_of, const int* zero_u0,
                                const float* initial_state, void* o, float* final_state,
                                void* stream);

/* ----------------------------------------------------------------------------------
 * Packed ("varlen") gated-delta prefill: n_seqs sequences of different lengths back to back
 * on one token axis, one call.  Replaces the per-sequence loop around chunk_gated_delta_rule
 * in the reference's packed prefill (inference/models/atma.py:494-503; the loop is named as
 * the remaining prefill gap in docs/kernel.md:328-329) and follows the cu_seqlens convention
 * of flash-linear-attention's chunk_gated_delta_rule.
 *   q [total][H][dk]; k, v [total][Hkv][d]; g, beta fp32 [total][H]; o [total][H][dv]
 *   cu_seqlens   DEVICE int32 [n_seqs + 1], token offsets (cu_seqlens[n_seqs] <= total)
 *   state: EITHER dense arrays initial_state / final_state fp32 [n_seqs][H][dk][dv] (each
 *   may be NULL: start from zero / do not return), OR a slot-indexed table state_table
 *   ([rows][H][dk][dv] fp32, slot_stride elements between rows) with DEVICE int64 slots
 *   [n_seqs]: sequence i starts from row slots[i] when has_initial is NULL or
 *   has_initial[i] != 0 (DEVICE int32), else from zero, and its final state is written to
 *   that row in place.  A sequence of length 0 leaves its state unchanged.
 *   16-bit inputs with dk = dv = 128 only (ATMA_ERR_INVALID otherwise: loop over
 *   atma_gated_delta_scan).  scratch: atma_gated_delta_scan_varlen_scratch_bytes bytes,
 *   256-byte aligned.  No host synchronisation; safe to capture in a CUDA graph.
 * ---------------------------------------------------------------------------------- */
int atma_gated_delta_scan_varlen(const void* q, const void* k, const void* v, int dtype,
                                 const float* g, const float* beta, const int32_t* cu_seqlens,
                                 int n_seqs, int64_t total_tokens, const float* initial_state,
                                 float* final_state, float* state_table, int64_t slot_stride,
                                 const int64_t* slots, const int32_t* has_initial, void* o,
                                 void* scratch, int H, int Hkv, int dk, int dv, int normalize_qk,
                                 float scale, void* stream);
int64_t atma_gated_delta_scan_varlen_scratch_bytes(int64_t total_tokens, int n_seqs, int H,
                                                   int dk, int dv);

/* The packed prefill with state snapshots for prefix reuse (the reference's engine shares K/V
 * pages across requests but restarts the memory state from zero, docs/inference.md:72-75,
 * inference/models/atma.py:477-479; a state saved at page boundaries makes the reuse exact).
 * As atma_gated_delta_scan_varlen with a state table, plus: after every snap_every_tokens tokens
 * (a multiple of 64, e.g. the cache page size) that lie wholly inside sequence i, the fp32 state
 * [H][dk][dv] is written to snapshots[snap_offsets[i] + j], j = 0, 1, ... (snap_offsets: DEVICE
 * int32 [n_seqs]; the caller sizes snapshots as sum_i floor(len_i / snap_every_tokens) rows). */
int atma_gated_delta_scan_varlen_snapshots(const void* q, const void* k, const void* v, int dtype,
                                           const float* g, const float* beta,
                                           const int32_t* cu_seqlens, int n_seqs, int64_t total_tokens,
                                           float* state_table, int64_t slot_stride, const int64_t* slots,
                                           const int32_t* has_initial, void* o, void* scratch,
                                           int H, int Hkv, int dk, int dv, int normalize_qk, float scale,
                                           float* snapshots, const int32_t* snap_offsets,
                                           int snap_every_tokens, void* stream);

/* ------------------------------------------------------------------------------------
 * Depthwise causal conv, one decode step, in place on a slot-indexed state table.
 * Replaces kernel/causal_conv1d_triton.py:17-42 behind causal_conv1d_decode_step (:46-63).
 * x, out [B][D] (row strides x_sb / out_sb), weight [D][K] dense, state [max_seqs][D][K-1]
 * with slot stride state_ss, all of dtype `dtype`; slots int64 [B].  K in 2..8.
 * ---------------------------------------------------------------------------------- */
int atma_causal_conv1d_decode_step(const void* x, int64_t x_sb, const void* weight,
                                   const int64_t* slots, void* state, int64_t state_ss,
                                   void* out, int64_t out_sb, int B, int D, int K,
                                   int dtype, void* stream);

/* ------------------------------------------------------------------------------------
 * Depthwise causal conv over packed ragged prompts + final-state write.
 * Replaces kernel/inference_ops_triton.py:17-63 behind packed_causal_conv1d (:139-160),
 * and the per-sequence conv of inference/models/atma.py:104-157.
 * x, out [tokens][C] (row strides), weight [C][K] dense, K in 2..4; per-token int32 maps
 * token_seq_start / token_seq_end / token_seq_slot.  state [max_seqs][C][K-1] receives the
 * last K-1 inputs of every sequence (zeros where the prompt is shorter).  init_state, if
 * not NULL, is a table of the same shape whose rows supply the left context instead of
 * zeros (a continuation chunk); it must not alias `state`.  residual != 0 adds x to the
 * result (the Canon form q + conv(q)).
 * ---------------------------------------------------------------------------------- */
int atma_packed_causal_conv1d(const void* x, int64_t x_st, const void* weight,
                              void* out, int64_t out_st,
                              void* state, const void* init_state, int64_t state_ss,
                              const int32_t* token_seq_start, const int32_t* token_seq_end,
                              const int32_t* token_seq_slot,
                              int total, int C, int K, int dtype, int residual, void* stream);

/* ----------------------------------------------------------------------------------
 * Fused q/k/v preparation of a global layer's packed prefill (next-step fusion; the reference
 * runs it as separate ops: F.rms_norm of q and k per head, x + packed_causal_conv1d(x) for
 * q, k and v, then store_kvcache - inference/models/atma.py:391-399,431-441,468-471).
 *   q_gate  [total][H][..]: q is the first dk elements of each head's chunk (element strides
 *           qg_row_stride / qg_head_stride; the gate half is not touched)
 *   k, v    [total][Hkv][dk] with row strides in elements
 *   w_*     conv weights [C][K] in the activation dtype, K in 2..4
 *   state_* conv-state tables [rows][C][K-1], row stride state_*_stride elements: the row
 *           token_seq_slot of a sequence receives its last K-1 conv inputs (NULL = not kept)
 *   init_*  tables of the same layout read as the left context of every sequence with a
 *           slot >= 0 (a continued prefix); NULL = fresh prompts.  Must not alias state_*.
 *   token_seq_start / _end / _slot: DEVICE int32 per token, as for atma_packed_causal_conv1d
 *   q_out [total][H][dk], k_out, v_out [total][Hkv][dk] dense
 *   k_cache, v_cache [slots][Hkv][dk] + DEVICE int64 slot_mapping per token (-1 = skip);
 *           NULL caches = no scatter.   eps: the RMSNorm epsilon (F.rms_norm with eps=None uses
 *           the fp32 machine epsilon, also for 16-bit inputs).  Each fused op rounds to the activation dtype where the
 *           separate ops would.
 * ---------------------------------------------------------------------------------- */
int atma_qkv_prep_prefill(const void* q_gate, int64_t qg_row_stride, int64_t qg_head_stride,
                          const void* k, int64_t k_row_stride, const void* v, int64_t v_row_stride,
                          const void* w_q, const void* w_k, const void* w_v,
                          void* state_q, void* state_k, void* state_v,
                          const void* init_q, const void* init_k, const void* init_v,
                          int64_t state_q_stride, int64_t state_k_stride, int64_t state_v_stride,
                          const int32_t* token_seq_start, const int32_t* token_seq_end,
                          const int32_t* token_seq_slot, void* q_out, void* k_out, void* v_out,
                          void* k_cache, void* v_cache, const int64_t* slot_mapping,
                          int total, int H, int Hkv, int dk, int K, float eps, int dtype, void* stream);

/* ----------------------------------------------------------------------------------
 * Gate epilogues of a global layer's mixing output (next-step fusions; the reference runs each
 * as three eager ops).
 * atma_sigmoid_gate_mul: out[r][h][c] = x[r][h][c] * sigmoid(gate[r][h][c]) - the
 *   `c_flat * torch.sigmoid(gate)` of `_combine` (inference/models/atma.py:552-558).  x and gate
 *   with (row, head) element strides, so the gate half of the q|gate projection is read in place
 *   and c may be the (tokens, H, dk) or the (H, tokens, dk) layout; out dense [rows][H][dk].
 * atma_rms_sigmoid_gate: out[r][h*dk+c] = RMSNorm_dk(x[r][h][:])[c] * sigmoid(gate[r][h*dk+c])
 *   - the memory read-out `F.rms_norm(r, (dk,)) * torch.sigmoid(mem.gate(x))`
 *   (inference/models/atma.py:373-375; model/blocks.py:486-489).  x dense [rows][H][dk], gate
 *   [rows][H*dk] with a row stride; affine-free norm; dk <= 128.
 * Both round to the activation dtype after the sigmoid, after the norm and after the product,
 * as the separate ops do.  head_dim a multiple of 8; pointers 16-byte aligned.
 * ---------------------------------------------------------------------------------- */
int atma_sigmoid_gate_mul(const void* x, int64_t x_row_stride, int64_t x_head_stride,
                          const void* gate, int64_t gate_row_stride, int64_t gate_head_stride,
                          void* out, int rows, int H, int dk, int dtype, void* stream);
int atma_rms_sigmoid_gate(const void* x, const void* gate, int64_t gate_row_stride, void* out,
                          int rows, int H, int dk, float eps, int dtype, void* stream);

/* ----------------------------------------------------------------------------------
 * Gated short convolution of the local (LFM2) layers, fused around the depthwise conv:
 *   projected = in_proj(x) = [B | C | x'] (row of 3*D);  y = C * conv(B * x')
 * (inference/models/atma.py:631-673: chunk, B*x', _gpu_conv_step / packed_causal_conv1d, C*conv).
 * _decode_step: one token per sequence; state [rows][D][K-1] updated in place at DEVICE int64
 *   slots (slot < 0: no state is read or written), holds the last K-1 GATED inputs, oldest first.
 * _packed: ragged prefill with the per-token maps of atma_packed_causal_conv1d; each sequence's
 *   row of `state` receives its last K-1 gated inputs; init_state (same layout, must not alias
 *   state) is the left context of every sequence with a slot >= 0, NULL = fresh prompts.
 * out [rows][D]; weight [D][K], K in 2..4; strides in elements.
 * ---------------------------------------------------------------------------------- */
int atma_lfm2_conv_decode_step(const void* projected, int64_t proj_row_stride, const void* weight,
                               const int64_t* slots, void* state, int64_t state_slot_stride,
                               void* out, int64_t out_row_stride, int B, int D, int K, int dtype,
                               void* stream);
int atma_lfm2_conv_packed(const void* projected, int64_t proj_row_stride, const void* weight,
                          void* out, int64_t out_row_stride, void* state, const void* init_state,
                          int64_t state_slot_stride, const int32_t* token_seq_start,
                          const int32_t* token_seq_end, const int32_t* token_seq_slot,
                          int total, int D, int K, int dtype, void* stream);

/* ------------------------------------------------------------------------------------
 * Scatter new K/V rows into the paged cache.  Replaces inference/layers/attention.py:7-27
 * behind store_kvcache (:30-56).  key, value [N][D] with row strides (D = Hkv*dk
 * contiguous); caches are flat [slots][D]; slot_mapping int32 [N], -1 skips the row.
 * ---------------------------------------------------------------------------------- */
int atma_store_kvcache(const void* key, int64_t key_stride, const void* value, int64_t value_stride,
                       void* k_cache, void* v_cache, const int32_t* slot_mapping,
                       int N, int D, int elem_size, void* stream);

/* ------------------------------------------------------------------------------------
 * gate * relu(x)^2 with eager-bf16 rounding of the square.
 * Replaces kernel/inference_ops_triton.py:102-120 behind squared_relu_gate (:124-135).
 * x, gate [rows][width] with row strides (columns contiguous); out dense.
 * ---------------------------------------------------------------------------------- */
int atma_squared_relu_gate(const void* x, int64_t x_stride, const void* gate, int64_t gate_stride,
                           void* out, int rows, int width, int dtype, void* stream);

/* 15 x / sqrt(x^2 + 225) with eager-bf16 rounding after each op.
 * Replaces kernel/inference_ops_triton.py:194-211 behind softcap_logits (:215-223). */
int atma_softcap_logits(const void* x, void* out, int64_t n, int dtype, void* stream);

/* ------------------------------------------------------------------------------------
 * Projection + affine-free per-head RMSNorm.  Replaces the prototype
 * kernel/inference_ops_triton.py:65-100 behind linear_head_rms (:164-189).
 * x [M][K] dense, weight [heads*width][K] dense, bias [heads*width] or NULL, out
 * [M][heads*width]; width = head_dim * (gated ? 2 : 1); only the first head_dim columns
 * of each head are normalised.
 * ---------------------------------------------------------------------------------- */
int atma_linear_head_rms(const void* x, const void* weight, const void* bias, void* out,
                         int M, int K, int heads, int head_dim, int gated, float eps,
                         int dtype, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* ATMA_B200_H_ */
