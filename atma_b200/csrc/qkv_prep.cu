// Fused q/k/v preparation for the packed prefill of a global layer: per-head RMSNorm of q and k,
// the three depthwise causal "Canon" convolutions in residual form (x + conv(x)) over packed
// variable-length sequences with their conv-state rows, and the scatter of the post-conv K and V
// rows into the paged cache - one pass over the projections instead of the reference's
// rms_norm x2, packed_causal_conv1d x3, residual add x3 and store_kvcache
// (inference/models/atma.py:396-399,431-441,468-471; kernel/inference_ops_triton.py:139-160;
// inference/layers/attention.py:30-56).
//
// Sixteen threads cover a head row with eight channels each (16-byte accesses); such a group holds
// 8 tokens plus the K-1 rows before them in registers, reduces the row sums of squares with
// shuffles and writes every output once.  The eight groups of a CTA take up to eight heads of the
// SAME tokens, so that a CTA touches whole token rows (neighbouring DRAM pages) rather than one
// 256-byte piece per 4 KB.  The kernel is bandwidth-bound: each projection element comes from DRAM
// once (the K-1 halo rows of a tile are its neighbour's rows, i.e. cache hits) and q, k, v plus
// the K/V cache rows go out once.
#include "common.cuh"

namespace atma {

namespace {

constexpr int kPrepTok = 8;        // tokens per 16-thread group
constexpr int kPrepGroups = 8;     // groups per CTA
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
  int nq, upc_q, upc_kv;                             // q-head chunks in grid.y; heads per chunk (1, 2, 4 or 8) for q and for k|v
  float eps;
};

// eight consecutive channels per thread: one 16-byte access for 16-bit types, two for fp32
template <typename T> __device__ __forceinline__ void load8(const T* p, float (&o)[8]);
template <> __device__ __forceinline__ void load8<float>(const float* p, float (&o)[8]) {
  const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
  o[0] = a.x; o[1] = a.y; o[2] = a.z; o[3] = a.w; o[4] = b.x; o[5] = b.y; o[6] = b.z; o[7] = b.w;
}
template <> __device__ __forceinline__ void load8<__nv_bfloat16>(const __nv_bfloat16* p, float (&o)[8]) {
  const uint4 u = *reinterpret_cast<const uint4*>(p);
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) { const float2 f = __bfloat1622float2(h[i]); o[2 * i] = f.x; o[2 * i + 1] = f.y; }
}
template <> __device__ __forceinline__ void load8<__half>(const __half* p, float (&o)[8]) {
  const uint4 u = *reinterpret_cast<const uint4*>(p);
  const __half2* h = reinterpret_cast<const __half2*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) { const float2 f = __half22float2(h[i]); o[2 * i] = f.x; o[2 * i + 1] = f.y; }
}
template <typename T> __device__ __forceinline__ void store8(T* p, const float (&v)[8]);
template <> __device__ __forceinline__ void store8<float>(float* p, const float (&v)[8]) {
  *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
  *reinterpret_cast<float4*>(p + 4) = make_float4(v[4], v[5], v[6], v[7]);
}
template <> __device__ __forceinline__ void store8<__nv_bfloat16>(__nv_bfloat16* p, const float (&v)[8]) {
  uint4 u;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
  *reinterpret_cast<uint4*>(p) = u;
}
template <> __device__ __forceinline__ void store8<__half>(__half* p, const float (&v)[8]) {
  uint4 u;
  __half2* h = reinterpret_cast<__half2*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2half2_rn(v[2 * i], v[2 * i + 1]);
  *reinterpret_cast<uint4*>(p) = u;
}

template <typename T, int K>
__global__ void __launch_bounds__(128, 3)
qkv_prep_kernel(const PrepArgs a) {
  constexpr int kCtaTok = kPrepTok * kPrepGroups;                // at most this many tokens per CTA
  __shared__ int s_s0[kCtaTok], s_e0[kCtaTok], s_slot[kCtaTok];
  __shared__ long long s_cs[kCtaTok];
  const int grp = threadIdx.x >> 4, li = threadIdx.x & 15;      // 16 threads x 8 channels cover one head row
  // blockIdx.y < nq: a chunk of q heads; else a chunk of the 2*Hkv k and v heads.  The `upc` heads of a
  // chunk sit side by side in the CTA (their rows of one token are neighbours in memory); with fewer
  // than 8 heads per chunk the other groups take further 8-token tiles.
  const bool is_q = (int)blockIdx.y < a.nq;
  const int chunk = is_q ? blockIdx.y : blockIdx.y - a.nq;
  const int n_units = is_q ? a.H : 2 * a.Hkv;
  const int upc = is_q ? a.upc_q : a.upc_kv, tpc = kPrepGroups / upc;
  const int unit = chunk * upc + grp % upc;
  const int cta_t0 = blockIdx.x * tpc * kPrepTok;
  const int t0 = cta_t0 + (grp / upc) * kPrepTok;
  if (threadIdx.x < tpc * kPrepTok) {                            // the per-token maps of the CTA's tokens
    const int t = cta_t0 + threadIdx.x;
    const bool ok = t < a.total;
    s_s0[threadIdx.x] = ok ? a.seq_start[t] : 0;
    s_e0[threadIdx.x] = ok ? a.seq_end[t] : 0;
    s_slot[threadIdx.x] = ok ? a.seq_slot[t] : -1;
    s_cs[threadIdx.x] = (ok && a.slot_mapping != nullptr) ? a.slot_mapping[t] : -1;
  }
  const int which = is_q ? 0 : (unit < a.Hkv ? 1 : 2);
  const int head = is_q ? unit : (unit < a.Hkv ? unit : unit - a.Hkv);
  const int heads = is_q ? a.H : a.Hkv;
  const int c = li * 8;
  const bool active = c < a.dk && unit < n_units && t0 < a.total;
  const bool normalize = which != 2;

  const T* src; int64_t row_st;
  if (which == 0) { src = (const T*)a.qg + (int64_t)head * a.qg_head; row_st = a.qg_row; }
  else if (which == 1) { src = (const T*)a.k + (int64_t)head * a.dk; row_st = a.k_row; }
  else { src = (const T*)a.v + (int64_t)head * a.dk; row_st = a.v_row; }
  T* dst = (T*)(which == 0 ? a.q_out : (which == 1 ? a.k_out : a.v_out)) + (int64_t)head * a.dk;
  const int64_t dst_row = (int64_t)heads * a.dk;
  const int ch = head * a.dk + c;                                // first of this thread's conv channels

  float wt[8][K];
#pragma unroll
  for (int j = 0; j < 8; ++j)
#pragma unroll
    for (int kk = 0; kk < K; ++kk)
      wt[j][kk] = active ? to_f32(((const T*)a.w[which])[(int64_t)(ch + j) * K + kk]) : 0.f;

  // ---- rows t0-(K-1) .. t0+kPrepTok-1, normalised ------------------------------------------------------
  float x[kPrepTok + K - 1][8];
#pragma unroll
  for (int i = 0; i < kPrepTok + K - 1; ++i) {
    const int t = t0 - (K - 1) + i;
    if (active && t >= 0 && t < a.total) load8<T>(src + (int64_t)t * row_st + c, x[i]);
    else {
#pragma unroll
      for (int j = 0; j < 8; ++j) x[i][j] = 0.f;
    }
  }
  if (normalize) {
    const float inv_dk = 1.0f / (float)a.dk;
#pragma unroll
    for (int i = 0; i < kPrepTok + K - 1; ++i) {
      float ss = 0.f;
#pragma unroll
      for (int j = 0; j < 8; ++j) ss = fmaf(x[i][j], x[i][j], ss);
#pragma unroll
      for (int o = 8; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);     // the 16 threads of the row
      const float r = rsqrtf(ss * inv_dk + a.eps);
#pragma unroll
      for (int j = 0; j < 8; ++j) x[i][j] = round_through<T>(x[i][j] * r);           // the eager op rounds to T here
    }
  }
  __syncthreads();                                               // the token maps are in shared memory
  if (!active) return;

  T* state = (T*)a.state[which];
  const T* init = (const T*)a.init[which];
  const int64_t state_ss = a.state_ss[which];
  T* cache = (T*)(which == 1 ? a.k_cache : a.v_cache);

#pragma unroll
  for (int i = 0; i < kPrepTok; ++i) {
    const int t = t0 + i;
    if (t >= a.total) break;
    const int ti = t - cta_t0;
    const int s0 = s_s0[ti], e0 = s_e0[ti], slot = s_slot[ti];
    const bool from_state = init != nullptr && slot >= 0;
    // channel j's input `back` rows before token t as this sequence sees it: its own rows, else
    // its saved state, else 0
    auto tap = [&](int back, int j) -> float {
      if (t - back >= s0) return x[i + (K - 1) - back][j];
      if (from_state) return to_f32(init[slot * state_ss + (int64_t)(ch + j) * (K - 1) + (K - 1) - (s0 - (t - back))]);
      return 0.f;
    };
    float y[8];
    if (t - (K - 1) >= s0) {                                     // the common case: all taps inside the sequence
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        float acc = 0.f;
#pragma unroll
        for (int kk = 0; kk < K; ++kk) acc = fmaf(x[i + kk][j], wt[j][kk], acc);
        y[j] = x[i + K - 1][j] + round_through<T>(acc);          // x + conv(x), the conv rounded as eager does
      }
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        float acc = 0.f;
#pragma unroll
        for (int kk = 0; kk < K; ++kk) acc = fmaf(tap(K - 1 - kk, j), wt[j][kk], acc);
        y[j] = x[i + K - 1][j] + round_through<T>(acc);
      }
    }
    store8<T>(dst + (int64_t)t * dst_row + c, y);
    if (which != 0) {
      const int64_t cs = s_cs[ti];
      if (cs >= 0) store8<T>(cache + (cs * a.Hkv + head) * a.dk + c, y);
    }
    if (t == e0 - 1 && state != nullptr && slot >= 0) {
      // this token closes its sequence: persist its last K-1 conv inputs, oldest first
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        float keep[K - 1];
#pragma unroll
        for (int kk = 0; kk < K - 1; ++kk) keep[kk] = tap(K - 2 - kk, j);
#pragma unroll
        for (int kk = 0; kk < K - 1; ++kk) state[slot * state_ss + (int64_t)(ch + j) * (K - 1) + kk] = from_f32<T>(keep[kk]);
      }
    }
  }
}

template <typename T>
int launch_prep(const PrepArgs& a, cudaStream_t st) {
  const int tok_q = kPrepGroups / a.upc_q * kPrepTok, tok_kv = kPrepGroups / a.upc_kv * kPrepTok;
  const int nx = ((a.total + tok_q - 1) / tok_q > (a.total + tok_kv - 1) / tok_kv) ? (a.total + tok_q - 1) / tok_q
                                                                                     : (a.total + tok_kv - 1) / tok_kv;
  dim3 grid(nx, a.nq + (2 * a.Hkv + a.upc_kv - 1) / a.upc_kv), block(128);
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
  ATMA_REQUIRE(H > 0 && Hkv > 0 && dk > 0 && dk <= 128 && dk % 8 == 0,
               "qkv_prep_prefill: needs head_dim <= 128 and a multiple of 8 (got %d)", dk);
  ATMA_REQUIRE(qg_row_stride % 8 == 0 && qg_head_stride % 8 == 0 && k_row_stride % 8 == 0 && v_row_stride % 8 == 0 &&
                   (uintptr_t)q_gate % 16 == 0 && (uintptr_t)k % 16 == 0 && (uintptr_t)v % 16 == 0 &&
                   (uintptr_t)q_out % 16 == 0 && (uintptr_t)k_out % 16 == 0 && (uintptr_t)v_out % 16 == 0 &&
                   (uintptr_t)k_cache % 16 == 0 && (uintptr_t)v_cache % 16 == 0,
               "qkv_prep_prefill: rows must be 16-byte aligned (pointers and strides in multiples of 8 elements)");
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
  auto pow2_at_most_8 = [](int n) { int p = 1; while (p < n && p < 8) p <<= 1; return p; };
  a.upc_q = pow2_at_most_8(H);
  a.upc_kv = pow2_at_most_8(2 * Hkv);
  a.nq = (H + a.upc_q - 1) / a.upc_q;
  int rc = ATMA_OK;
  ATMA_DISPATCH_DTYPE(dtype, T, { rc = launch_prep<T>(a, (cudaStream_t)stream); });
  return rc;
}
