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
// Thread = one channel x a run of TOK_PER_THREAD consecutive tokens; the last K-1 inputs slide
// through registers so x is read once.  Left context that falls before the token's own
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
