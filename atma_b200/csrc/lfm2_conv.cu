// The gated short convolution of the local (LFM2) layers, fused around the depthwise causal conv:
//   projected = in_proj(x) = [B | C | x'] ;  y = C * conv(B * x')
// (inference/models/atma.py:631-673).  The reference runs chunk, B*x', the conv (decode step or
// packed prefill) and C*conv as separate ops; here the projection is read once, the gated input
// B*x' never reaches memory (only its last K-1 values, the conv state), and y is written once.
// Rounding to the activation dtype happens where the separate ops round: after B*x', after the
// conv, after the product with C.
#include "common.cuh"

namespace atma {

namespace {

// ---- decode step: one token per sequence, in place on the slot-indexed state table -----------------
template <typename T, int K>
__global__ void lfm2_conv_step_kernel(const T* __restrict__ proj, int64_t proj_sb, const T* __restrict__ w,
                                      const int64_t* __restrict__ slots, T* __restrict__ state, int64_t state_ss,
                                      T* __restrict__ out, int64_t out_sb, int D) {
  const int b = blockIdx.x;
  const int d = blockIdx.y * blockDim.x + threadIdx.x;
  if (d >= D) return;
  const T* p = proj + b * proj_sb;
  const float bv = to_f32(p[d]), cv = to_f32(p[D + d]), xv = to_f32(p[2 * D + d]);
  const T xg = from_f32<T>(bv * xv);                            // the gated conv input, as eager materialises it
  const int64_t slot = slots[b];
  float acc = to_f32(xg) * to_f32(w[d * K + (K - 1)]);
  if (slot >= 0) {
    T* s = state + slot * state_ss + (int64_t)d * (K - 1);
    T old[K - 1];
#pragma unroll
    for (int j = 0; j < K - 1; ++j) old[j] = s[j];
#pragma unroll
    for (int j = 0; j < K - 1; ++j) acc = fmaf(to_f32(old[j]), to_f32(w[d * K + j]), acc);
#pragma unroll
    for (int j = 0; j + 1 < K - 1; ++j) s[j] = old[j + 1];
    s[K - 2] = xg;
  }
  out[b * out_sb + d] = from_f32<T>(cv * round_through<T>(acc));
}

// Wide form of the decode step (D a multiple of 8, 16-bit types, 16-byte aligned rows): a thread owns eight channels
// and asks for everything it needs up front - the B, C and x' pieces of the projection row, the 8 x K taps and the
// 8 x (K-1) state values, each a contiguous run - so a step is one round of loads, the arithmetic and one round of
// stores.  Same rounding points as the channel-per-thread form.
template <typename T, int K>
__global__ void __launch_bounds__(128)
lfm2_conv_step_wide_kernel(const T* __restrict__ proj, int64_t proj_sb, const T* __restrict__ w,
                           const int64_t* __restrict__ slots, T* __restrict__ state, int64_t state_ss,
                           T* __restrict__ out, int64_t out_sb, int D) {
  const int b = blockIdx.x;
  const int d0 = (blockIdx.y * blockDim.x + threadIdx.x) * 8;
  if (d0 >= D) return;
  union V8 { uint4 u; T e[8]; };
  const T* p = proj + b * proj_sb;
  V8 bv, cv, xv;
  bv.u = *reinterpret_cast<const uint4*>(p + d0);
  cv.u = *reinterpret_cast<const uint4*>(p + D + d0);
  xv.u = *reinterpret_cast<const uint4*>(p + 2 * D + d0);
  T wr[8 * K], sr[8 * (K - 1)], sn[8 * (K - 1)];
#pragma unroll
  for (int i = 0; i < K; ++i) reinterpret_cast<uint4*>(wr)[i] = *reinterpret_cast<const uint4*>(w + (int64_t)d0 * K + 8 * i);
  const int64_t slot = slots[b];
  T* st = slot >= 0 ? state + slot * state_ss + (int64_t)d0 * (K - 1) : nullptr;
  if (st != nullptr) {
#pragma unroll
    for (int i = 0; i < K - 1; ++i) reinterpret_cast<uint4*>(sr)[i] = *reinterpret_cast<const uint4*>(st + 8 * i);
  }
  V8 o;
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const T xg = from_f32<T>(to_f32(bv.e[j]) * to_f32(xv.e[j]));        // the gated conv input, as eager materialises it
    float acc = to_f32(xg) * to_f32(wr[j * K + K - 1]);
    if (st != nullptr) {
#pragma unroll
      for (int t = 0; t < K - 1; ++t) acc = fmaf(to_f32(sr[j * (K - 1) + t]), to_f32(wr[j * K + t]), acc);
#pragma unroll
      for (int t = 0; t + 1 < K - 1; ++t) sn[j * (K - 1) + t] = sr[j * (K - 1) + t + 1];
      sn[j * (K - 1) + K - 2] = xg;
    }
    o.e[j] = from_f32<T>(to_f32(cv.e[j]) * round_through<T>(acc));
  }
  if (st != nullptr) {
#pragma unroll
    for (int i = 0; i < K - 1; ++i) *reinterpret_cast<uint4*>(st + 8 * i) = reinterpret_cast<const uint4*>(sn)[i];
  }
  *reinterpret_cast<uint4*>(out + b * out_sb + d0) = o.u;
}

// ---- packed prefill: thread = one channel x a run of consecutive tokens ---------------------------------
constexpr int kLfmTokPerThread = 16;

template <typename T, int K>
__global__ void lfm2_conv_packed_kernel(const T* __restrict__ proj, int64_t proj_st, const T* __restrict__ w,
                                        T* __restrict__ out, int64_t out_st, T* __restrict__ state,
                                        const T* __restrict__ init_state, int64_t state_ss,
                                        const int32_t* __restrict__ seq_start, const int32_t* __restrict__ seq_end,
                                        const int32_t* __restrict__ seq_slot, int total, int D) {
  const int d = blockIdx.y * blockDim.x + threadIdx.x;
  const int t0 = blockIdx.x * kLfmTokPerThread;
  if (d >= D) return;
  float wt[K];
#pragma unroll
  for (int j = 0; j < K; ++j) wt[j] = to_f32(w[d * K + j]);
  auto gated = [&](int t) -> float {                            // B * x' of packed row t, rounded to T
    const T* p = proj + (int64_t)t * proj_st;
    return round_through<T>(to_f32(p[d]) * to_f32(p[2 * D + d]));
  };
  // the gated inputs of rows t0-(K-1) .. t0-1 (only used where they belong to the token's own sequence)
  float win[K];
#pragma unroll
  for (int j = 0; j < K - 1; ++j) {
    const int t = t0 - (K - 1) + j;
    win[j] = t >= 0 ? gated(t) : 0.f;
  }
  const int t1 = min(t0 + kLfmTokPerThread, total);
  for (int t = t0; t < t1; ++t) {
    const int s0 = seq_start[t], e0 = seq_end[t], slot = seq_slot[t];
    win[K - 1] = gated(t);
    // input `back` rows before t as this sequence sees it: its own rows, else its saved state, else 0
    auto tap = [&](int back) -> float {
      if (t - back >= s0) return win[K - 1 - back];
      if (init_state != nullptr && slot >= 0)
        return to_f32(init_state[slot * state_ss + (int64_t)d * (K - 1) + (K - 1) - (s0 - (t - back))]);
      return 0.f;
    };
    float acc = 0.f;
#pragma unroll
    for (int j = 0; j < K; ++j) acc = fmaf(tap(K - 1 - j), wt[j], acc);
    const float cv = to_f32(proj[(int64_t)t * proj_st + D + d]);
    out[(int64_t)t * out_st + d] = from_f32<T>(cv * round_through<T>(acc));
    if (t == e0 - 1 && slot >= 0 && state != nullptr) {
      float keep[K - 1];
#pragma unroll
      for (int j = 0; j < K - 1; ++j) keep[j] = tap(K - 2 - j);
#pragma unroll
      for (int j = 0; j < K - 1; ++j) state[slot * state_ss + (int64_t)d * (K - 1) + j] = from_f32<T>(keep[j]);
    }
#pragma unroll
    for (int j = 0; j < K - 1; ++j) win[j] = win[j + 1];
  }
}

// Vector form of the packed prefill (D and the row strides multiples of 16 bytes, 16-byte aligned bases): thread =
// 16 bytes of channels x a run of kLfmVecTok consecutive tokens.  The B and x' parts of all kLfmVecTok + K - 1 rows
// are requested as 16-byte loads up front and multiplied into the gated input once per row; the C part is read where
// the token is written.  Rows before a sequence start (saved state or zero) and the state write of a closing token
// are rare and out of line.  Same rounding points and accumulation order as the scalar form.
constexpr int kLfmVecTok = 4;

template <typename T> struct LfmVec16 {
  static constexpr int N = 16 / sizeof(T);
  union { uint4 u; T e[N]; };
};

template <typename T, int K>
__device__ __noinline__ uint4 lfm2_row_before_start(const T* __restrict__ init_state, int64_t base, int rows_before) {
  LfmVec16<T> r;
#pragma unroll
  for (int n = 0; n < LfmVec16<T>::N; ++n)
    r.e[n] = init_state != nullptr ? init_state[base + (int64_t)n * (K - 1) + (K - 1 - rows_before)] : from_f32<T>(0.f);
  return r.u;
}
template <typename T, int K>
__device__ __noinline__ void lfm2_state_write(T* __restrict__ dst, const uint4* keep) {
#pragma unroll
  for (int j = 0; j < K - 1; ++j) {
    LfmVec16<T> r;
    r.u = keep[j];
#pragma unroll
    for (int n = 0; n < LfmVec16<T>::N; ++n) dst[(int64_t)n * (K - 1) + j] = r.e[n];
  }
}

template <typename T, int K>
__global__ void __launch_bounds__(128, 3)
lfm2_conv_packed_vec_kernel(const T* __restrict__ proj, int64_t proj_st, const T* __restrict__ w, T* __restrict__ out,
                            int64_t out_st, T* __restrict__ state, const T* __restrict__ init_state, int64_t state_ss,
                            const int32_t* __restrict__ seq_start, const int32_t* __restrict__ seq_end,
                            const int32_t* __restrict__ seq_slot, int total, int D) {
  constexpr int N = LfmVec16<T>::N;
  const int groups = D / N;
  const int64_t gid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int cg = (int)(gid % groups);
  const int64_t run = gid / groups;
  if (run * kLfmVecTok >= total) return;
  const int t0 = (int)(run * kLfmVecTok);
  const int d0 = cg * N;
  const int nt = min(kLfmVecTok, total - t0);

  LfmVec16<T> bx[kLfmVecTok + K - 1], xx[kLfmVecTok + K - 1], cc[kLfmVecTok];
#pragma unroll
  for (int i = 0; i < kLfmVecTok + K - 1; ++i) {
    const int t = t0 - (K - 1) + i;
    if (t >= 0 && t < total) {
      const T* p = proj + (int64_t)t * proj_st + d0;
      bx[i].u = *reinterpret_cast<const uint4*>(p);
      xx[i].u = *reinterpret_cast<const uint4*>(p + 2 * D);
    } else {
      bx[i].u = make_uint4(0u, 0u, 0u, 0u);
      xx[i].u = make_uint4(0u, 0u, 0u, 0u);
    }
  }
#pragma unroll
  for (int i = 0; i < kLfmVecTok; ++i)
    cc[i].u = i < nt ? *reinterpret_cast<const uint4*>(proj + (int64_t)(t0 + i) * proj_st + D + d0) : make_uint4(0u, 0u, 0u, 0u);
  float wt[N][K];
  if ((K * (int)sizeof(T) * N) % 16 == 0 && (reinterpret_cast<uintptr_t>(w) & 15) == 0) {
    constexpr int kPieces = (N * K * (int)sizeof(T) + 15) / 16;     // the thread's N x K weights are neighbours in memory
    LfmVec16<T> wv[kPieces];
#pragma unroll
    for (int i = 0; i < kPieces; ++i) wv[i].u = *reinterpret_cast<const uint4*>(w + (int64_t)d0 * K + i * N);
#pragma unroll
    for (int n = 0; n < N; ++n)
#pragma unroll
      for (int j = 0; j < K; ++j) wt[n][j] = to_f32(wv[(n * K + j) / N].e[(n * K + j) % N]);
  } else {
#pragma unroll
    for (int n = 0; n < N; ++n)
#pragma unroll
      for (int j = 0; j < K; ++j) wt[n][j] = to_f32(w[(d0 + n) * K + j]);
  }
  // gated input B * x' of every row of the run, rounded to T as eager materialises it (reuses bx)
#pragma unroll
  for (int i = 0; i < kLfmVecTok + K - 1; ++i)
#pragma unroll
    for (int n = 0; n < N; ++n) bx[i].e[n] = from_f32<T>(to_f32(bx[i].e[n]) * to_f32(xx[i].e[n]));

  const int sa = seq_start[t0], ea = seq_end[t0 + nt - 1], sla = seq_slot[t0];
  const bool uniform = sa == seq_start[t0 + nt - 1] && ea > t0 + nt;   // one sequence, not closed inside the run
  if (uniform && sa <= t0 - (K - 1)) {
    // common case: the run and its K-1 rows of left context lie inside one sequence
    float win[K][N];
#pragma unroll
    for (int rl = 0; rl < kLfmVecTok + K - 1; ++rl) {
#pragma unroll
      for (int n = 0; n < N; ++n) win[rl % K][n] = to_f32(bx[rl].e[n]);
      if (rl >= K - 1 && rl - (K - 1) < nt) {
        LfmVec16<T> o;
#pragma unroll
        for (int n = 0; n < N; ++n) {
          float acc = 0.f;
#pragma unroll
          for (int j = 0; j < K; ++j) acc = fmaf(win[(rl - (K - 1) + j) % K][n], wt[n][j], acc);
          o.e[n] = from_f32<T>(to_f32(cc[rl - (K - 1)].e[n]) * round_through<T>(acc));
        }
        *reinterpret_cast<uint4*>(out + (int64_t)(t0 + rl - (K - 1)) * out_st + d0) = o.u;
      }
    }
    return;
  }
#pragma unroll 1
  for (int i = 0; i < nt; ++i) {
    const int t = t0 + i;
    const int s0 = uniform ? sa : seq_start[t], e0 = uniform ? ea : seq_end[t], sl = uniform ? sla : seq_slot[t];
    LfmVec16<T> prev[K];                              // prev[j] = gated input K-1-j rows before t as this sequence sees it
#pragma unroll
    for (int j = 0; j < K; ++j) {
      const int src = t - (K - 1 - j);
      if (src >= s0) {
        const int idx = i + j;                        // bx[] index; selected without dynamic register indexing
        uint4 u = bx[0].u;
#pragma unroll
        for (int q = 1; q < kLfmVecTok + K - 1; ++q) if (q == idx) u = bx[q].u;
        prev[j].u = u;
      } else {
        prev[j].u = lfm2_row_before_start<T, K>(sl >= 0 ? init_state : nullptr,
                                                (sl >= 0 ? sl * state_ss : 0) + (int64_t)d0 * (K - 1), s0 - src);
      }
    }
    uint4 cu = cc[0].u;
#pragma unroll
    for (int q = 1; q < kLfmVecTok; ++q) if (q == i) cu = cc[q].u;
    LfmVec16<T> cv, o;
    cv.u = cu;
#pragma unroll
    for (int n = 0; n < N; ++n) {
      float acc = 0.f;
#pragma unroll
      for (int j = 0; j < K; ++j) acc = fmaf(to_f32(prev[j].e[n]), wt[n][j], acc);
      o.e[n] = from_f32<T>(to_f32(cv.e[n]) * round_through<T>(acc));
    }
    *reinterpret_cast<uint4*>(out + (int64_t)t * out_st + d0) = o.u;
    if (t == e0 - 1 && sl >= 0 && state != nullptr) {
      uint4 keep[K - 1];
#pragma unroll
      for (int j = 0; j < K - 1; ++j) keep[j] = prev[j + 1].u;
      lfm2_state_write<T, K>(state + sl * state_ss + (int64_t)d0 * (K - 1), keep);
    }
  }
}

template <typename T>
int launch_lfm2_step(const void* proj, int64_t proj_sb, const void* w, const int64_t* slots, void* state,
                     int64_t state_ss, void* out, int64_t out_sb, int B, int D, int K, cudaStream_t st) {
  if constexpr (sizeof(T) == 2) {
    auto al = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
    if (D % 8 == 0 && proj_sb % 8 == 0 && out_sb % 8 == 0 && state_ss % 8 == 0 && al(proj) && al(w) && al(state) && al(out)) {
      dim3 wgrid(B, (D / 8 + 127) / 128), wblock(128);
      switch (K) {
        case 2: lfm2_conv_step_wide_kernel<T, 2><<<wgrid, wblock, 0, st>>>((const T*)proj, proj_sb, (const T*)w, slots, (T*)state, state_ss, (T*)out, out_sb, D); break;
        case 3: lfm2_conv_step_wide_kernel<T, 3><<<wgrid, wblock, 0, st>>>((const T*)proj, proj_sb, (const T*)w, slots, (T*)state, state_ss, (T*)out, out_sb, D); break;
        case 4: lfm2_conv_step_wide_kernel<T, 4><<<wgrid, wblock, 0, st>>>((const T*)proj, proj_sb, (const T*)w, slots, (T*)state, state_ss, (T*)out, out_sb, D); break;
        default: return fail(ATMA_ERR_UNSUPPORTED, "lfm2_conv_decode_step: kernel size %d not in 2..4", K);
      }
      return launch_status("lfm2_conv_decode_step");
    }
  }
  dim3 grid(B, (D + 255) / 256), block(256);
  switch (K) {
    case 2: lfm2_conv_step_kernel<T, 2><<<grid, block, 0, st>>>((const T*)proj, proj_sb, (const T*)w, slots, (T*)state, state_ss, (T*)out, out_sb, D); break;
    case 3: lfm2_conv_step_kernel<T, 3><<<grid, block, 0, st>>>((const T*)proj, proj_sb, (const T*)w, slots, (T*)state, state_ss, (T*)out, out_sb, D); break;
    case 4: lfm2_conv_step_kernel<T, 4><<<grid, block, 0, st>>>((const T*)proj, proj_sb, (const T*)w, slots, (T*)state, state_ss, (T*)out, out_sb, D); break;
    default: return fail(ATMA_ERR_UNSUPPORTED, "lfm2_conv_decode_step: kernel size %d not in 2..4", K);
  }
  return launch_status("lfm2_conv_decode_step");
}

template <typename T>
int launch_lfm2_packed(const void* proj, int64_t proj_st, const void* w, void* out, int64_t out_st, void* state,
                       const void* init_state, int64_t state_ss, const int32_t* s0, const int32_t* e0, const int32_t* sl,
                       int total, int D, int K, cudaStream_t st) {
  constexpr int N = 16 / (int)sizeof(T);
  if (D % N == 0 && proj_st % N == 0 && out_st % N == 0 && (reinterpret_cast<uintptr_t>(proj) & 15) == 0 &&
      (reinterpret_cast<uintptr_t>(out) & 15) == 0) {
    const int64_t threads = (int64_t)(D / N) * ((total + kLfmVecTok - 1) / kLfmVecTok);
    dim3 vgrid((unsigned)((threads + 127) / 128)), vblock(128);
    switch (K) {
      case 2: lfm2_conv_packed_vec_kernel<T, 2><<<vgrid, vblock, 0, st>>>((const T*)proj, proj_st, (const T*)w, (T*)out, out_st, (T*)state, (const T*)init_state, state_ss, s0, e0, sl, total, D); break;
      case 3: lfm2_conv_packed_vec_kernel<T, 3><<<vgrid, vblock, 0, st>>>((const T*)proj, proj_st, (const T*)w, (T*)out, out_st, (T*)state, (const T*)init_state, state_ss, s0, e0, sl, total, D); break;
      case 4: lfm2_conv_packed_vec_kernel<T, 4><<<vgrid, vblock, 0, st>>>((const T*)proj, proj_st, (const T*)w, (T*)out, out_st, (T*)state, (const T*)init_state, state_ss, s0, e0, sl, total, D); break;
      default: return fail(ATMA_ERR_UNSUPPORTED, "lfm2_conv_packed: kernel size %d not in 2..4", K);
    }
    return launch_status("lfm2_conv_packed");
  }
  dim3 grid((total + kLfmTokPerThread - 1) / kLfmTokPerThread, (D + 127) / 128), block(128);
#define ATMA_CASE(KK)                                                                                               \
  case KK:                                                                                                          \
    lfm2_conv_packed_kernel<T, KK><<<grid, block, 0, st>>>((const T*)proj, proj_st, (const T*)w, (T*)out, out_st,  \
                                                           (T*)state, (const T*)init_state, state_ss, s0, e0, sl,  \
                                                           total, D);                                               \
    break;
  switch (K) {
    ATMA_CASE(2) ATMA_CASE(3) ATMA_CASE(4)
    default: return fail(ATMA_ERR_UNSUPPORTED, "lfm2_conv_packed: kernel size %d not in 2..4", K);
  }
#undef ATMA_CASE
  return launch_status("lfm2_conv_packed");
}

}  // namespace
}  // namespace atma

using namespace atma;

extern "C" int atma_lfm2_conv_decode_step(const void* projected, int64_t proj_row_stride, const void* weight,
                                          const int64_t* slots, void* state, int64_t state_slot_stride, void* out,
                                          int64_t out_row_stride, int B, int D, int K, int dtype, void* stream) {
  ATMA_REQUIRE(dtype_ok(dtype), "lfm2_conv_decode_step: unsupported dtype %d", dtype);
  if (B <= 0 || D <= 0) return ATMA_OK;
  ATMA_REQUIRE(slots != nullptr && state != nullptr, "lfm2_conv_decode_step: slots and the state table are required");
  int rc = ATMA_OK;
  ATMA_DISPATCH_DTYPE(dtype, T, {
    rc = launch_lfm2_step<T>(projected, proj_row_stride, weight, slots, state, state_slot_stride, out, out_row_stride, B, D, K,
                             (cudaStream_t)stream);
  });
  return rc;
}

extern "C" int atma_lfm2_conv_packed(const void* projected, int64_t proj_row_stride, const void* weight, void* out,
                                     int64_t out_row_stride, void* state, const void* init_state,
                                     int64_t state_slot_stride, const int32_t* token_seq_start,
                                     const int32_t* token_seq_end, const int32_t* token_seq_slot, int total, int D,
                                     int K, int dtype, void* stream) {
  ATMA_REQUIRE(dtype_ok(dtype), "lfm2_conv_packed: unsupported dtype %d", dtype);
  ATMA_REQUIRE(init_state == nullptr || init_state != state, "lfm2_conv_packed: init_state must not alias state");
  if (total <= 0 || D <= 0) return ATMA_OK;
  ATMA_REQUIRE(token_seq_start && token_seq_end && token_seq_slot, "lfm2_conv_packed: the per-token sequence arrays are required");
  int rc = ATMA_OK;
  ATMA_DISPATCH_DTYPE(dtype, T, {
    rc = launch_lfm2_packed<T>(projected, proj_row_stride, weight, out, out_row_stride, state, init_state, state_slot_stride,
                               token_seq_start, token_seq_end, token_seq_slot, total, D, K, (cudaStream_t)stream);
  });
  return rc;
}
