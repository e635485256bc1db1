// Depthwise causal convolution: the one-token decode step (in place on a slot-indexed
// state table) and the packed ragged prefill with its final-state write.
#include "common.cuh"

namespace atma {

// ---- decode step -------------------------------------------------------------------------
// out[b,d] = sum_{j<K-1} w[d,j] * state[slot,d,j] + w[d,K-1] * x[b,d]; state shifts left by
// one and takes x.  One thread owns one channel, so the in-place shift has no hazard.
template <typename T, int K>
__global__ void conv_step_kernel(const T* __restrict__ x, int64_t x_sb, const T* __restrict__ w,
                                 const int64_t* __restrict__ slots, T* __restrict__ state,
                                 int64_t state_ss, T* __restrict__ out, int64_t out_sb, int D) {
  const int b = blockIdx.x;
  const int d = blockIdx.y * blockDim.x + threadIdx.x;
  if (d >= D) return;
  const int64_t slot = slots[b];
  const T xv = x[b * x_sb + d];
  float acc = to_f32(xv) * to_f32(w[d * K + (K - 1)]);
  if (slot >= 0) {
    T* s = state + slot * state_ss + (int64_t)d * (K - 1);
    T old[K - 1];
#pragma unroll
    for (int j = 0; j < K - 1; ++j) old[j] = s[j];
#pragma unroll
    for (int j = 0; j < K - 1; ++j) acc = fmaf(to_f32(old[j]), to_f32(w[d * K + j]), acc);
#pragma unroll
    for (int j = 0; j + 1 < K - 1; ++j) s[j] = old[j + 1];
    s[K - 2] = xv;
  }
  out[b * out_sb + d] = from_f32<T>(acc);
}

// ---- packed prefill ------------------------------------------------------------------------
// Scalar form (any channel count, stride or alignment): thread = one channel x a run of
// kConvTokPerThread consecutive tokens.  Left context that falls before the token's own
// sequence start is zero (fresh prompt) or comes from init_state (continuation chunk).
constexpr int kConvTokPerThread = 16;

template <typename T, int K>
__global__ void packed_conv_kernel(const T* __restrict__ x, int64_t x_st, const T* __restrict__ w,
                                   T* __restrict__ out, int64_t out_st, T* __restrict__ state,
                                   const T* __restrict__ init_state, int64_t state_ss,
                                   const int32_t* __restrict__ seq_start,
                                   const int32_t* __restrict__ seq_end,
                                   const int32_t* __restrict__ seq_slot, int total, int C,
                                   int residual) {
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  const int t0 = blockIdx.x * kConvTokPerThread;
  if (c >= C) return;
  float wt[K];
#pragma unroll
  for (int j = 0; j < K; ++j) wt[j] = to_f32(w[c * K + j]);

  // fetch the input at packed row `src` as seen from a token whose sequence starts at `s0`
  auto fetch = [&](int src, int s0, int slot) -> T {
    if (src >= s0) return x[(int64_t)src * x_st + c];
    if (init_state != nullptr && slot >= 0) {
      const int back = s0 - src;                       // 1 .. K-1 rows before the chunk
      return init_state[slot * state_ss + (int64_t)c * (K - 1) + (K - 1 - back)];
    }
    return from_f32<T>(0.f);
  };

  const int t1 = min(t0 + kConvTokPerThread, total);
  for (int t = t0; t < t1; ++t) {
    const int s0 = seq_start[t], e0 = seq_end[t], slot = seq_slot[t];
    float acc = 0.f;
    T cur = x[(int64_t)t * x_st + c];
#pragma unroll
    for (int j = 0; j < K - 1; ++j) {
      const int src = t - (K - 1 - j);
      acc = fmaf(to_f32(fetch(src, s0, slot)), wt[j], acc);
    }
    acc = fmaf(to_f32(cur), wt[K - 1], acc);
    if (residual) acc += to_f32(cur);
    out[(int64_t)t * out_st + c] = from_f32<T>(acc);
    if (t == e0 - 1 && slot >= 0) {
      // this token closes its sequence: persist the last K-1 inputs, oldest first
#pragma unroll
      for (int j = 0; j < K - 1; ++j) {
        const int src = e0 - (K - 1) + j;
        state[slot * state_ss + (int64_t)c * (K - 1) + j] = fetch(src, s0, slot);
      }
    }
  }
}

// Vector form (channel count and row strides multiples of 16 bytes, 16-byte aligned bases): thread =
// 16 bytes of channels (8 for the 2-byte types, 4 for fp32) x a run of kVecTok consecutive tokens.
// All kVecTok + K - 1 rows of the run are requested as 16-byte loads before the first use, so a thread
// keeps 11 loads in flight and every input row is read once from memory (the K-1 rows of overlap with
// the neighbouring run hit L2); the taps then index registers.  A run that lies inside one sequence and
// does not close it skips the per-token sequence maps.  Same accumulation order as the scalar form.
constexpr int kVecTok = 8;                          // tokens per group (all loads of a group in flight together)
constexpr int kVecGroups = 4;                       // consecutive groups per thread

template <typename T> struct Vec16 {
  static constexpr int N = 16 / sizeof(T);
  union { uint4 u; T e[N]; };
};

// The rare rows of the vector form, kept out of line so that the common path stays small: a row that lies
// before the sequence start (from init_state, channel-major [C][K-1], or zero), and the state write of a
// token that closes its sequence.
template <typename T, int K>
__device__ __noinline__ uint4 conv_row_before_start(const T* __restrict__ init_state, int64_t base, int rows_before) {
  Vec16<T> r;
#pragma unroll
  for (int n = 0; n < Vec16<T>::N; ++n)
    r.e[n] = init_state != nullptr ? init_state[base + (int64_t)n * (K - 1) + (K - 1 - rows_before)] : from_f32<T>(0.f);
  return r.u;
}
template <typename T, int K>
__device__ __noinline__ void conv_state_write(T* __restrict__ dst, const uint4* keep) {
#pragma unroll
  for (int j = 0; j < K - 1; ++j) {
    Vec16<T> r;
    r.u = keep[j];
#pragma unroll
    for (int n = 0; n < Vec16<T>::N; ++n) dst[(int64_t)n * (K - 1) + j] = r.e[n];
  }
}

template <typename T, int K>
__global__ void __launch_bounds__(128, 4)
packed_conv_vec_kernel(const T* __restrict__ x, int64_t x_st, const T* __restrict__ w, T* __restrict__ out,
                       int64_t out_st, T* __restrict__ state, const T* __restrict__ init_state, int64_t state_ss,
                       const int32_t* __restrict__ seq_start, const int32_t* __restrict__ seq_end,
                       const int32_t* __restrict__ seq_slot, int total, int C, int residual) {
  constexpr int N = Vec16<T>::N;
  const int groups = C / N;
  const int64_t gid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int cg = (int)(gid % groups);
  const int64_t run = gid / groups;
  if (run * (kVecTok * kVecGroups) >= total) return;
  const int c0 = cg * N;
  // the thread's N x K weights are neighbours in memory ([C][K]): N*K*sizeof(T) bytes as 16-byte loads
  float wt[N][K];
  {
    constexpr int kPieces = N * K * (int)sizeof(T) / 16;            // = K
    Vec16<T> wv[kPieces];
#pragma unroll
    for (int i = 0; i < kPieces; ++i) wv[i].u = *reinterpret_cast<const uint4*>(w + (int64_t)c0 * K + i * N);
#pragma unroll
    for (int n = 0; n < N; ++n)
#pragma unroll
      for (int j = 0; j < K; ++j) wt[n][j] = to_f32(wv[(n * K + j) / N].e[(n * K + j) % N]);
  }
  // The thread walks kVecGroups consecutive groups of kVecTok tokens; after a group that lay inside one sequence its
  // last K-1 rows are still in registers (fp32) and serve as the next group's left context.
  float prevw[K - 1][N];
  bool have_prev = false;
#pragma unroll 1
  for (int gi = 0; gi < kVecGroups; ++gi) {
  const int64_t t0l = (run * kVecGroups + gi) * kVecTok;
  if (t0l >= total) break;
  const int t0 = (int)t0l;
  const int nt = min(kVecTok, total - t0);
  const int sa = seq_start[t0], ea = seq_end[t0 + nt - 1], sla = seq_slot[t0];
  const bool uniform = sa == seq_start[t0 + nt - 1] && ea > t0 + nt;   // one sequence, not closed inside the group
  if (uniform && nt == kVecTok && sa <= t0 - (K - 1)) {
    // common case: the group and its K-1 rows of left context lie inside one sequence
    Vec16<T> cur[kVecTok];
#pragma unroll
    for (int i = 0; i < kVecTok; ++i) cur[i].u = *reinterpret_cast<const uint4*>(x + (int64_t)(t0 + i) * x_st + c0);
    if (!have_prev) {
#pragma unroll
      for (int j = 0; j < K - 1; ++j) {
        Vec16<T> h;
        h.u = *reinterpret_cast<const uint4*>(x + (int64_t)(t0 - (K - 1) + j) * x_st + c0);
#pragma unroll
        for (int n = 0; n < N; ++n) prevw[j][n] = to_f32(h.e[n]);
      }
    }
#pragma unroll
    for (int i = 0; i < kVecTok; ++i) {
      Vec16<T> o;
      float xc[N];
#pragma unroll
      for (int n = 0; n < N; ++n) {
        xc[n] = to_f32(cur[i].e[n]);
        float acc = 0.f;
#pragma unroll
        for (int j = 0; j < K - 1; ++j) acc = fmaf(prevw[j][n], wt[n][j], acc);
        acc = fmaf(xc[n], wt[n][K - 1], acc);
        if (residual) acc += xc[n];
        o.e[n] = from_f32<T>(acc);
      }
      *reinterpret_cast<uint4*>(out + (int64_t)(t0 + i) * out_st + c0) = o.u;
#pragma unroll
      for (int j = 0; j + 1 < K - 1; ++j)
#pragma unroll
        for (int n = 0; n < N; ++n) prevw[j][n] = prevw[j + 1][n];
#pragma unroll
      for (int n = 0; n < N; ++n) prevw[K - 2][n] = xc[n];
    }
    have_prev = true;
    continue;
  }
  have_prev = false;
  Vec16<T> rows[kVecTok + K - 1];                     // rows[i] = packed row t0 - (K-1) + i
#pragma unroll
  for (int i = 0; i < kVecTok + K - 1; ++i) {
    const int t = t0 - (K - 1) + i;
    if (t >= 0 && t < total) rows[i].u = *reinterpret_cast<const uint4*>(x + (int64_t)t * x_st + c0);
    else rows[i].u = make_uint4(0u, 0u, 0u, 0u);
  }
#pragma unroll 1
  for (int i = 0; i < nt; ++i) {
    const int t = t0 + i;
    const int s0 = uniform ? sa : seq_start[t], e0 = uniform ? ea : seq_end[t], sl = uniform ? sla : seq_slot[t];
    Vec16<T> prev[K];                                 // prev[j] = the input K-1-j rows before t as this sequence sees it
#pragma unroll
    for (int j = 0; j < K; ++j) {
      const int src = t - (K - 1 - j);
      if (src >= s0) {
        const int idx = i + j;                        // rows[] index; selected without dynamic register indexing
        uint4 u = rows[0].u;
#pragma unroll
        for (int q = 1; q < kVecTok + K - 1; ++q) if (q == idx) u = rows[q].u;
        prev[j].u = u;
      } else {
        prev[j].u = conv_row_before_start<T, K>(sl >= 0 ? init_state : nullptr,
                                                (sl >= 0 ? sl * state_ss : 0) + (int64_t)c0 * (K - 1), s0 - src);
      }
    }
    Vec16<T> o;
#pragma unroll
    for (int n = 0; n < N; ++n) {
      float acc = 0.f;
#pragma unroll
      for (int j = 0; j < K; ++j) acc = fmaf(to_f32(prev[j].e[n]), wt[n][j], acc);
      if (residual) acc += to_f32(prev[K - 1].e[n]);
      o.e[n] = from_f32<T>(acc);
    }
    *reinterpret_cast<uint4*>(out + (int64_t)t * out_st + c0) = o.u;
    if (t == e0 - 1 && sl >= 0) {                     // closes its sequence: keep the last K-1 inputs, oldest first
      uint4 keep[K - 1];
#pragma unroll
      for (int j = 0; j < K - 1; ++j) keep[j] = prev[j + 1].u;
      conv_state_write<T, K>(state + sl * state_ss + (int64_t)c0 * (K - 1), keep);
    }
  }
  }                                                   // next group of the thread
}

template <typename T>
bool conv_vec_ok(const void* x, int64_t x_st, const void* w, const void* out, int64_t out_st, int C) {
  constexpr int N = 16 / sizeof(T);
  return C % N == 0 && x_st % N == 0 && out_st % N == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0 &&
         (reinterpret_cast<uintptr_t>(w) & 15) == 0 && (reinterpret_cast<uintptr_t>(out) & 15) == 0;
}

template <typename T>
int launch_conv_step(const void* x, int64_t x_sb, const void* w, const int64_t* slots, void* state,
                     int64_t state_ss, void* out, int64_t out_sb, int B, int D, int K,
                     cudaStream_t st) {
  dim3 grid(B, (D + 255) / 256), block(256);
#define ATMA_CASE(KK)                                                                          \
  case KK:                                                                                     \
    conv_step_kernel<T, KK><<<grid, block, 0, st>>>((const T*)x, x_sb, (const T*)w, slots,     \
                                                    (T*)state, state_ss, (T*)out, out_sb, D);  \
    break;
  switch (K) {
    ATMA_CASE(2) ATMA_CASE(3) ATMA_CASE(4) ATMA_CASE(5) ATMA_CASE(6) ATMA_CASE(7) ATMA_CASE(8)
    default: return fail(ATMA_ERR_UNSUPPORTED, "causal_conv1d_decode_step: kernel size %d not in 2..8", K);
  }
#undef ATMA_CASE
  return launch_status("causal_conv1d_decode_step");
}

template <typename T>
int launch_packed_conv(const void* x, int64_t x_st, const void* w, void* out, int64_t out_st,
                       void* state, const void* init_state, int64_t state_ss,
                       const int32_t* s0, const int32_t* e0, const int32_t* sl, int total, int C,
                       int K, int residual, cudaStream_t st) {
  if (conv_vec_ok<T>(x, x_st, w, out, out_st, C)) {
    const int64_t threads = (int64_t)(C / (16 / (int)sizeof(T))) * ((total + kVecTok * kVecGroups - 1) / (kVecTok * kVecGroups));
    dim3 grid((unsigned)((threads + 127) / 128)), block(128);
    switch (K) {
      case 2: packed_conv_vec_kernel<T, 2><<<grid, block, 0, st>>>((const T*)x, x_st, (const T*)w, (T*)out, out_st, (T*)state, (const T*)init_state, state_ss, s0, e0, sl, total, C, residual); break;
      case 3: packed_conv_vec_kernel<T, 3><<<grid, block, 0, st>>>((const T*)x, x_st, (const T*)w, (T*)out, out_st, (T*)state, (const T*)init_state, state_ss, s0, e0, sl, total, C, residual); break;
      case 4: packed_conv_vec_kernel<T, 4><<<grid, block, 0, st>>>((const T*)x, x_st, (const T*)w, (T*)out, out_st, (T*)state, (const T*)init_state, state_ss, s0, e0, sl, total, C, residual); break;
      default: return fail(ATMA_ERR_UNSUPPORTED, "packed_causal_conv1d: kernel size %d not in 2..4", K);
    }
    return launch_status("packed_causal_conv1d");
  }
  dim3 grid((total + kConvTokPerThread - 1) / kConvTokPerThread, (C + 127) / 128), block(128);
#define ATMA_CASE(KK)                                                                            \
  case KK:                                                                                       \
    packed_conv_kernel<T, KK><<<grid, block, 0, st>>>((const T*)x, x_st, (const T*)w, (T*)out,   \
                                                      out_st, (T*)state, (const T*)init_state,   \
                                                      state_ss, s0, e0, sl, total, C, residual); \
    break;
  switch (K) {
    ATMA_CASE(2) ATMA_CASE(3) ATMA_CASE(4)
    default: return fail(ATMA_ERR_UNSUPPORTED, "packed_causal_conv1d: kernel size %d not in 2..4", K);
  }
#undef ATMA_CASE
  return launch_status("packed_causal_conv1d");
}

}  // namespace atma

using namespace atma;

extern "C" int atma_causal_conv1d_decode_step(const void* x, int64_t x_sb, const void* weight,
                                              const int64_t* slots, void* state, int64_t state_ss,
                                              void* out, int64_t out_sb, int B, int D, int K,
                                              int dtype, void* stream) {
  ATMA_REQUIRE(dtype_ok(dtype), "causal_conv1d_decode_step: unsupported dtype %d", dtype);
  if (B <= 0 || D <= 0) return ATMA_OK;
  int rc = ATMA_OK;
  ATMA_DISPATCH_DTYPE(dtype, T, {
    rc = launch_conv_step<T>(x, x_sb, weight, slots, state, state_ss, out, out_sb, B, D, K,
                             (cudaStream_t)stream);
  });
  return rc;
}

extern "C" int atma_packed_causal_conv1d(const void* x, int64_t x_st, const void* weight, void* out,
                                         int64_t out_st, void* state, const void* init_state,
                                         int64_t state_ss, const int32_t* token_seq_start,
                                         const int32_t* token_seq_end,
                                         const int32_t* token_seq_slot, int total, int C, int K,
                                         int dtype, int residual, void* stream) {
  ATMA_REQUIRE(dtype_ok(dtype), "packed_causal_conv1d: unsupported dtype %d", dtype);
  ATMA_REQUIRE(init_state == nullptr || init_state != state,
               "packed_causal_conv1d: init_state must not alias state");
  if (total <= 0 || C <= 0) return ATMA_OK;
  int rc = ATMA_OK;
  ATMA_DISPATCH_DTYPE(dtype, T, {
    rc = launch_packed_conv<T>(x, x_st, weight, out, out_st, state, init_state, state_ss,
                               token_seq_start, token_seq_end, token_seq_slot, total, C, K,
                               residual, (cudaStream_t)stream);
  });
  return rc;
}
