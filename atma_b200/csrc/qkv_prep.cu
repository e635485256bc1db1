// Fused q/k/v preparation for the packed prefill of a global layer: per-head RMSNorm of q and k,
// the three depthwise causal "Canon" convolutions in residual form (x + conv(x)) over packed
// variable-length sequences with their conv-state rows, and the scatter of the post-conv K and V
// rows into the paged cache - one pass over the projections instead of the reference's
// rms_norm x2, packed_causal_conv1d x3, residual add x3 and store_kvcache
// (inference/models/atma.py:396-399,431-441,468-471; kernel/inference_ops_triton.py:139-160;
// inference/layers/attention.py:30-56).
//
// One CTA = one head (of q, k or v) x a tile of 32 tokens.  Thread c owns channel c of the head:
// it holds the tile's inputs (plus the K-1 rows before the tile) in registers, the row sums of
// squares are reduced across the CTA through shared memory, and every output is written once.
// The kernel is bandwidth-bound: it reads each projection element once (a (K-1)/32 halo aside)
// and writes q, k, v once plus the K/V cache rows.
#include "common.cuh"

namespace atma {

namespace {

constexpr int kPrepTok = 32;       // tokens per CTA
constexpr int kPrepMaxK = 4;

struct PrepArgs {
  const void* qg; int64_t qg_row, qg_head;          // q at the start of each head's chunk (the gate follows it)
  const void* k; int64_t k_row;
  const void* v; int64_t v_row;
  const void* w[3];                                  // [C][K] conv weights of q, k, v
  void* state[3]; int64_t state_ss[3];               // [rows][C][K-1] conv-state tables, written (may be null)
  const void* init[3];                               // same layout, read as left context (null = fresh sequences)
  const int32_t* seq_start; const int32_t* seq_end; const int32_t* seq_slot;   // per token
  void* q_out; void* k_out; void* v_out;             // dense [total][heads][dk]
  void* k_cache; void* v_cache; const int64_t* slot_mapping;   // cache rows [slot][Hkv][dk]; may be null
  int total, H, Hkv, dk, K;
  float eps;
};

template <typename T, int K>
__global__ void __launch_bounds__(128)
qkv_prep_kernel(const PrepArgs a) {
  __shared__ float s_part[kPrepTok + kPrepMaxK - 1][4];
  const int c = threadIdx.x, lane = c & 31, warp = c >> 5;
  const int t0 = blockIdx.x * kPrepTok;
  const int unit = blockIdx.y;                       // [0,H): q heads, [H,H+Hkv): k heads, then v heads
  const int which = unit < a.H ? 0 : (unit < a.H + a.Hkv ? 1 : 2);
  const int head = which == 0 ? unit : (which == 1 ? unit - a.H : unit - a.H - a.Hkv);
  const int heads = which == 0 ? a.H : a.Hkv;
  const bool active = c < a.dk;
  const bool normalize = which != 2;

  const T* src; int64_t row_st;
  if (which == 0) { src = (const T*)a.qg + (int64_t)head * a.qg_head; row_st = a.qg_row; }
  else if (which == 1) { src = (const T*)a.k + (int64_t)head * a.dk; row_st = a.k_row; }
  else { src = (const T*)a.v + (int64_t)head * a.dk; row_st = a.v_row; }
  T* dst = (T*)(which == 0 ? a.q_out : (which == 1 ? a.k_out : a.v_out)) + (int64_t)head * a.dk;
  const int64_t dst_row = (int64_t)heads * a.dk;
  const int ch = head * a.dk + c;                    // channel of the conv / state table

  // ---- inputs of rows t0-(K-1) .. t0+31 and their sums of squares ---------------------------------
  float x[kPrepTok + K - 1];
#pragma unroll
  for (int i = 0; i < kPrepTok + K - 1; ++i) {
    const int t = t0 - (K - 1) + i;
    x[i] = (active && t >= 0 && t < a.total) ? to_f32(src[(int64_t)t * row_st + c]) : 0.f;
  }
  if (normalize) {
#pragma unroll
    for (int i = 0; i < kPrepTok + K - 1; ++i) {
      const float s = warp_sum(x[i] * x[i]);
      if (lane == 0) s_part[i][warp] = s;
    }
    __syncthreads();
    const float inv_dk = 1.0f / (float)a.dk;
#pragma unroll
    for (int i = 0; i < kPrepTok + K - 1; ++i) {
      const float ss = s_part[i][0] + s_part[i][1] + s_part[i][2] + s_part[i][3];
      x[i] = round_through<T>(x[i] * rsqrtf(ss * inv_dk + a.eps));      // the eager op rounds to T here
    }
  }
  if (!active) return;

  float wt[K];
#pragma unroll
  for (int j = 0; j < K; ++j) wt[j] = to_f32(((const T*)a.w[which])[(int64_t)ch * K + j]);
  T* state = (T*)a.state[which];
  const T* init = (const T*)a.init[which];
  const int64_t state_ss = a.state_ss[which];

#pragma unroll
  for (int i = 0; i < kPrepTok; ++i) {
    const int t = t0 + i;
    if (t >= a.total) break;
    const int s0 = a.seq_start[t], e0 = a.seq_end[t], slot = a.seq_slot[t];
    const bool from_state = init != nullptr && slot >= 0;
    // input `back` rows before token t as this sequence sees it: its own rows, else its saved state, else 0
    auto tap = [&](int back) -> float {
      if (t - back >= s0) return x[i + (K - 1) - back];
      if (from_state) return to_f32(init[slot * state_ss + (int64_t)ch * (K - 1) + (K - 1) - (s0 - (t - back))]);
      return 0.f;
    };
    float acc = 0.f;
#pragma unroll
    for (int j = 0; j < K; ++j) acc = fmaf(tap(K - 1 - j), wt[j], acc);
    const T y = from_f32<T>(x[i + K - 1] + round_through<T>(acc));      // x + conv(x), each rounded as eager does
    dst[(int64_t)t * dst_row + c] = y;
    if (which != 0 && a.slot_mapping != nullptr) {
      const int64_t cs = a.slot_mapping[t];
      if (cs >= 0) ((T*)(which == 1 ? a.k_cache : a.v_cache))[(cs * a.Hkv + head) * a.dk + c] = y;
    }
    if (t == e0 - 1 && state != nullptr && slot >= 0) {
      // this token closes its sequence: persist its last K-1 conv inputs, oldest first
      float keep[K - 1];
#pragma unroll
      for (int j = 0; j < K - 1; ++j) keep[j] = tap(K - 2 - j);
#pragma unroll
      for (int j = 0; j < K - 1; ++j) state[slot * state_ss + (int64_t)ch * (K - 1) + j] = from_f32<T>(keep[j]);
    }
  }
}

template <typename T>
int launch_prep(const PrepArgs& a, cudaStream_t st) {
  dim3 grid((a.total + kPrepTok - 1) / kPrepTok, a.H + 2 * a.Hkv), block(128);
  switch (a.K) {
    case 2: qkv_prep_kernel<T, 2><<<grid, block, 0, st>>>(a); break;
    case 3: qkv_prep_kernel<T, 3><<<grid, block, 0, st>>>(a); break;
    default: qkv_prep_kernel<T, 4><<<grid, block, 0, st>>>(a); break;
  }
  return launch_status("qkv_prep_prefill");
}

}  // namespace
}  // namespace atma

using namespace atma;

extern "C" int atma_qkv_prep_prefill(const void* q_gate, int64_t qg_row_stride, int64_t qg_head_stride,
                                     const void* k, int64_t k_row_stride, const void* v, int64_t v_row_stride,
                                     const void* w_q, const void* w_k, const void* w_v, void* state_q,
                                     void* state_k, void* state_v, const void* init_q, const void* init_k,
                                     const void* init_v, int64_t state_q_stride, int64_t state_k_stride,
                                     int64_t state_v_stride, const int32_t* token_seq_start,
                                     const int32_t* token_seq_end, const int32_t* token_seq_slot,
                                     void* q_out, void* k_out, void* v_out,
                                     void* k_cache, void* v_cache, const int64_t* slot_mapping, int total, int H,
                                     int Hkv, int dk, int K, float eps, int dtype, void* stream) {
  ATMA_REQUIRE(dtype_ok(dtype), "qkv_prep_prefill: unsupported dtype %d", dtype);
  ATMA_REQUIRE(H > 0 && Hkv > 0 && dk > 0 && dk <= 128, "qkv_prep_prefill: needs head_dim <= 128 (got %d)", dk);
  ATMA_REQUIRE(K >= 2 && K <= kPrepMaxK, "qkv_prep_prefill: kernel size %d not in 2..4", K);
  ATMA_REQUIRE(token_seq_start && token_seq_end && token_seq_slot, "qkv_prep_prefill: the per-token sequence arrays are required");
  ATMA_REQUIRE((k_cache == nullptr) == (v_cache == nullptr), "qkv_prep_prefill: pass both caches or neither");
  ATMA_REQUIRE((init_q == nullptr || init_q != state_q) && (init_k == nullptr || init_k != state_k) &&
                   (init_v == nullptr || init_v != state_v),
               "qkv_prep_prefill: an initial-state table must not alias the table that is written");
  if (total <= 0) return ATMA_OK;
  PrepArgs a{};
  a.qg = q_gate; a.qg_row = qg_row_stride; a.qg_head = qg_head_stride;
  a.k = k; a.k_row = k_row_stride; a.v = v; a.v_row = v_row_stride;
  a.w[0] = w_q; a.w[1] = w_k; a.w[2] = w_v;
  a.state[0] = state_q; a.state[1] = state_k; a.state[2] = state_v;
  a.state_ss[0] = state_q_stride; a.state_ss[1] = state_k_stride; a.state_ss[2] = state_v_stride;
  a.seq_start = token_seq_start; a.seq_end = token_seq_end; a.seq_slot = token_seq_slot;
  a.init[0] = init_q; a.init[1] = init_k; a.init[2] = init_v;
  a.q_out = q_out; a.k_out = k_out; a.v_out = v_out;
  a.k_cache = k_cache; a.v_cache = v_cache; a.slot_mapping = k_cache ? slot_mapping : nullptr;
  a.total = total; a.H = H; a.Hkv = Hkv; a.dk = dk; a.K = K; a.eps = eps;
  int rc = ATMA_OK;
  ATMA_DISPATCH_DTYPE(dtype, T, { rc = launch_prep<T>(a, (cudaStream_t)stream); });
  return rc;
}
