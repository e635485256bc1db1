// Fused q/k/v preparation for the packed prefill of a global layer: per-head RMSNorm of q and k,
// the three depthwise causal "Canon" convolutions in residual form (x + conv(x)) over packed
// variable-length sequences with their conv-state rows, and the scatter of the post-conv K and V
// rows into the paged cache - one pass over the projections instead of the reference's
// rms_norm x2, packed_causal_conv1d x3, residual add x3 and store_kvcache
// (inference/models/atma.py:396-399,431-441,468-471; kernel/inference_ops_triton.py:139-160;
// inference/layers/attention.py:30-56).
//
// One CTA = 16 tokens x up to eight heads (of q, or of k and v).  The tile, plus the K-1 rows
// before it, is staged in shared memory with 16-byte asynchronous copies (whole token rows, so
// neighbouring DRAM pages).  A group of 16 threads x 8 channels then walks a run of consecutive
// tokens of one head: each row is read from the tile once, normalised in registers (row sums by
// shuffles), kept in a K-row register window for the taps, and q, k, v and the cache rows are
// written once.  Runs that lie inside one sequence take a straight-line path without per-row
// branches.  Four CTAs per SM (39 KB of shared memory, 128 registers each) overlap one tile's
// copies with another's arithmetic; each projection element comes from DRAM once (the K-1 halo
// rows of a tile are its neighbour's rows, i.e. cache hits) and every output goes out once.
#include <algorithm>

#include "common.cuh"
#include "mma_sync.cuh"

namespace atma {

namespace {

constexpr int kPrepTok = 16;       // tokens per CTA
constexpr int kPrepHeads = 8;      // heads per CTA (the rows of one token are neighbours in memory)
constexpr int kPrepThreads = 128;   // 8 groups of 16 threads: eight heads x one run of 16 tokens
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
  int nq;                                            // q-head chunks in grid.y (the k|v chunks follow)
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
// eight 16-bit values held in a uint4 register quad -> fp32
template <typename T> __device__ __forceinline__ void unpack8(const uint4& u, float (&o)[8]) {
  const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    if constexpr (std::is_same<T, __nv_bfloat16>::value) {
      o[2 * i] = __uint_as_float(w[i] << 16);
      o[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    } else {
      const __half2 h = *reinterpret_cast<const __half2*>(&w[i]);
      const float2 f = __half22float2(h);
      o[2 * i] = f.x; o[2 * i + 1] = f.y;
    }
  }
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

// round eight fp32 values through T and back, two per conversion instruction for the 16-bit types
template <typename T> __device__ __forceinline__ void round8(float (&v)[8]) {
  if constexpr (std::is_same<T, __nv_bfloat16>::value) {
#pragma unroll
    for (int i = 0; i < 4; ++i) { const float2 f = __bfloat1622float2(__floats2bfloat162_rn(v[2 * i], v[2 * i + 1])); v[2 * i] = f.x; v[2 * i + 1] = f.y; }
  } else if constexpr (std::is_same<T, __half>::value) {
#pragma unroll
    for (int i = 0; i < 4; ++i) { const float2 f = __half22float2(__floats2half2_rn(v[2 * i], v[2 * i + 1])); v[2 * i] = f.x; v[2 * i + 1] = f.y; }
  }
}

// The same on channel pairs: the straight-line path keeps a row as four float2 so that its multiplies, adds and
// fused multiply-adds issue as packed two-lane fp32 instructions (each lane rounds exactly as the scalar form).
template <typename T> __device__ __forceinline__ void unpack8(const uint4& u, float2 (&o)[4]) {
  float f[8];
  unpack8<T>(u, f);
#pragma unroll
  for (int i = 0; i < 4; ++i) o[i] = make_float2(f[2 * i], f[2 * i + 1]);
}
template <typename T> __device__ __forceinline__ void round8(float2 (&v)[4]) {
  if constexpr (std::is_same<T, __nv_bfloat16>::value) {
#pragma unroll
    for (int i = 0; i < 4; ++i) v[i] = __bfloat1622float2(__floats2bfloat162_rn(v[i].x, v[i].y));
  } else if constexpr (std::is_same<T, __half>::value) {
#pragma unroll
    for (int i = 0; i < 4; ++i) v[i] = __half22float2(__floats2half2_rn(v[i].x, v[i].y));
  }
}
template <typename T> __device__ __forceinline__ void store8(T* p, const float2 (&v)[4]) {
  static_assert(sizeof(T) == 2, "pairs are stored for the 16-bit types only");
  uint4 u;
  if constexpr (std::is_same<T, __nv_bfloat16>::value) {
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[i].x, v[i].y);
  } else {
    __half2* h = reinterpret_cast<__half2*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2half2_rn(v[i].x, v[i].y);
  }
  *reinterpret_cast<uint4*>(p) = u;
}

// 16-byte asynchronous copy global -> shared; src_bytes = 0 zero-fills the destination
__device__ __forceinline__ void prep_cp_async16(void* smem_dst, const void* gsrc, bool valid) {
  const uint32_t d = static_cast<uint32_t>(__cvta_generic_to_shared(smem_dst));
  const int n = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(gsrc), "r"(n) : "memory");
}

// A run of RUN consecutive tokens of one head that needs no sequence-boundary handling: rows come
// from the shared tile, the last K normalised rows stay in registers, outputs go out once.
template <typename T, int K, int RUN>
__device__ __forceinline__ void prep_plain_run(const T* trow, int row_elems, const float (&wt)[8][K], bool normalize,
                                               float inv_dk, float eps, uint32_t half_mask, T* dst, int64_t dst_row,
                                               T* cache, int64_t cache_row, const long long* s_cs) {
  long long cs[RUN];
#pragma unroll
  for (int i = 0; i < RUN; ++i) cs[i] = s_cs != nullptr ? s_cs[i] : -1;
  float win[K][8];
#pragma unroll
  for (int rl = 0; rl < RUN + K - 1; ++rl) {
    float (&x)[8] = win[rl % K];
    load8<T>(trow + rl * row_elems, x);
    if (normalize) {
      float ss = 0.f;
#pragma unroll
      for (int j = 0; j < 8; ++j) ss = fmaf(x[j], x[j], ss);
#pragma unroll
      for (int o = 8; o > 0; o >>= 1) ss += __shfl_xor_sync(half_mask, ss, o, 16);
      const float rs = rsqrtf(ss * inv_dk + eps);
#pragma unroll
      for (int j = 0; j < 8; ++j) x[j] *= rs;
      round8<T>(x);                                              // the eager op rounds to T here
    }
    if (rl >= K - 1) {
      const int i = rl - (K - 1);
      float y[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        float acc = 0.f;
#pragma unroll
        for (int kk = 0; kk < K; ++kk) acc = fmaf(win[(rl - (K - 1) + kk) % K][j], wt[j][kk], acc);
        y[j] = acc;
      }
      round8<T>(y);                                              // the conv rounded as eager does, then x + conv(x)
#pragma unroll
      for (int j = 0; j < 8; ++j) y[j] += x[j];
      store8<T>(dst + i * dst_row, y);
      if (cs[i] >= 0) store8<T>(cache + cs[i] * cache_row, y);
    }
  }
}

template <typename T, int K>
__global__ void __launch_bounds__(kPrepThreads, 4)
qkv_prep_kernel(const PrepArgs a) {
  // shared tile: rows t0-(K-1) .. t0+kPrepTok-1 of the chunk's (up to 8) heads, [row][head][dk] in T
  extern __shared__ __align__(16) uint8_t prep_smem[];
  T* tile = reinterpret_cast<T*>(prep_smem);
  __shared__ int s_s0[kPrepTok], s_e0[kPrepTok], s_slot[kPrepTok];
  __shared__ long long s_cs[kPrepTok];
  constexpr int kRows = kPrepTok + K - 1;
  constexpr int kVec = 16 / (int)sizeof(T);                      // elements per 16-byte piece
  const int tid = threadIdx.x;
  // blockIdx.y < nq: a chunk of q heads; else a chunk of the 2*Hkv k and v heads
  const bool is_q = (int)blockIdx.y < a.nq;
  const int chunk = is_q ? blockIdx.y : blockIdx.y - a.nq;
  const int n_units = is_q ? a.H : 2 * a.Hkv;
  const int u0 = chunk * kPrepHeads;
  const int nu = min(kPrepHeads, n_units - u0);                  // heads in this CTA
  const int t0 = blockIdx.x * kPrepTok;
  const int dk = a.dk, row_elems = kPrepHeads * dk;
  const int pieces = dk / kVec;                                  // 16-byte pieces per head row

  auto unit_src = [&](int u, const T*& src, int64_t& row_st, int& which, int& head) {
    if (is_q) { which = 0; head = u; src = (const T*)a.qg + (int64_t)head * a.qg_head; row_st = a.qg_row; }
    else if (u < a.Hkv) { which = 1; head = u; src = (const T*)a.k + (int64_t)head * dk; row_st = a.k_row; }
    else { which = 2; head = u - a.Hkv; src = (const T*)a.v + (int64_t)head * dk; row_st = a.v_row; }
  };

  // ---- stage the tile: every 16-byte piece by one asynchronous copy (whole rows per pass of the CTA) ---
  {
    const int per_row = nu * pieces;                              // 16-byte pieces per tile row (<= 256)
    const int rows_per_pass = kPrepThreads / per_row;
    const int r_off = tid / per_row, j = tid - r_off * per_row;
    const int ul = j / pieces, pc = j - ul * pieces;
    if (r_off < rows_per_pass) {
      const T* src; int64_t row_st; int which, head;
      unit_src(u0 + ul, src, row_st, which, head);
      src += pc * kVec;
      T* dst = tile + ul * dk + pc * kVec;
      for (int r = r_off; r < kRows; r += rows_per_pass) {
        const int t = t0 - (K - 1) + r;
        const bool ok = t >= 0 && t < a.total;
        prep_cp_async16(dst + r * row_elems, src + (ok ? (int64_t)t * row_st : 0), ok);
      }
    }
  }
  asm volatile("cp.async.commit_group;" ::: "memory");
  if (tid < kPrepTok) {                                          // the per-token maps of the CTA's tokens
    const int t = t0 + tid;
    const bool ok = t < a.total;
    s_s0[tid] = ok ? a.seq_start[t] : 0;
    s_e0[tid] = ok ? a.seq_end[t] : 0;
    s_slot[tid] = ok ? a.seq_slot[t] : -1;
    s_cs[tid] = (ok && a.slot_mapping != nullptr) ? a.slot_mapping[t] : -1;
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");
  __syncthreads();

  // ---- each 16-thread group walks a run of consecutive tokens of one head: the last K normalised
  //      rows stay in registers, so every tile row is read (and normalised) once per group ---------------
  const int grp = tid >> 4, li = tid & 15;                      // 16 threads x 8 channels cover one head row
  constexpr int kGroups = kPrepThreads / 16;
  const int gph = kGroups / nu;                                  // groups per head (2 with eight heads)
  const int ul = grp % nu, part = grp / nu;
  const int tpg = (kPrepTok + gph - 1) / gph;                    // tokens per group (<= 16)
  const int i_begin = part * tpg, i_end = min(kPrepTok, i_begin + tpg);
  const int c = li * 8;
  const bool lane_on = c < dk;
  const uint32_t half_mask = 0xffffu << (16 * (grp & 1));       // the two head rows of a warp are independent
  if (part >= gph || i_begin >= i_end) return;

  const T* src_unused; int64_t row_st_unused; int which, head;
  unit_src(u0 + ul, src_unused, row_st_unused, which, head);
  const bool normalize = which != 2;
  const int heads = which == 0 ? a.H : a.Hkv;
  const int ch = head * dk + c;                                  // first of this thread's conv channels
  T* state = (T*)a.state[which];
  const T* init = (const T*)a.init[which];
  const int64_t state_ss = a.state_ss[which];
  T* dst = (T*)(which == 0 ? a.q_out : (which == 1 ? a.k_out : a.v_out)) + head * dk + c;
  T* cache = (which == 0 || a.k_cache == nullptr) ? nullptr : (T*)(which == 1 ? a.k_cache : a.v_cache) + head * dk + c;
  const int64_t dst_row = (int64_t)heads * dk, cache_row = (int64_t)a.Hkv * dk;
  const float inv_dk = 1.0f / (float)dk;

  float wt[8][K];
#pragma unroll
  for (int j = 0; j < 8; ++j)
#pragma unroll
    for (int kk = 0; kk < K; ++kk) wt[j][kk] = lane_on ? to_f32(((const T*)a.w[which])[(int64_t)(ch + j) * K + kk]) : 0.f;

  const T* trow = tile + i_begin * row_elems + ul * dk + c;      // tile row i_begin <-> token t0 + i_begin - (K-1)
  float win[K][8];
  constexpr int kMaxRows = kPrepTok + K - 1;

  // ---- fast path: a full run (16 tokens with eight heads per CTA, 8 with four) that lies inside one
  //      sequence, not at its start or end: straight-line code, so the rows' load -> reduce -> scale
  //      chains overlap.  Both head rows of a warp share the code, so the decision is per warp. -----------
  {
    const int run = i_end - i_begin;
    const int t_first = t0 + i_begin, t_last = t_first + run - 1;
    const bool plain = (run == 16 || run == 8) && t_last < a.total && lane_on && s_s0[i_begin] <= t_first - (K - 1) &&
                       s_e0[i_begin] > t_last + 1 && s_s0[i_begin] == s_s0[i_begin + run - 1];
    const unsigned active = __activemask();
    if (__all_sync(active, plain)) {
      const long long* cs = cache != nullptr ? s_cs + i_begin : nullptr;
      if (run == 16)
        prep_plain_run<T, K, 16>(trow, row_elems, wt, normalize, inv_dk, a.eps, half_mask, dst + t_first * dst_row, dst_row,
                                 cache, cache_row, cs);
      else
        prep_plain_run<T, K, 8>(trow, row_elems, wt, normalize, inv_dk, a.eps, half_mask, dst + t_first * dst_row, dst_row,
                                cache, cache_row, cs);
      return;
    }
  }
#pragma unroll
  for (int rl = 0; rl < kMaxRows; ++rl) {
    if (rl >= i_end - i_begin + K - 1) break;
    float (&x)[8] = win[rl % K];
    if (lane_on) load8<T>(trow + rl * row_elems, x);
    else {
#pragma unroll
      for (int j = 0; j < 8; ++j) x[j] = 0.f;
    }
    if (normalize) {
      float ss = 0.f;
#pragma unroll
      for (int j = 0; j < 8; ++j) ss = fmaf(x[j], x[j], ss);
#pragma unroll
      for (int o = 8; o > 0; o >>= 1) ss += __shfl_xor_sync(half_mask, ss, o, 16);
      const float rs = rsqrtf(ss * inv_dk + a.eps);
#pragma unroll
      for (int j = 0; j < 8; ++j) x[j] = round_through<T>(x[j] * rs);                // the eager op rounds to T here
    }
    if (rl < K - 1 || !lane_on) continue;                        // still filling the window
    const int i = i_begin + rl - (K - 1);
    const int t = t0 + i;
    if (t >= a.total) break;
    const int s0 = s_s0[i], e0 = s_e0[i], slot = s_slot[i];
    const bool from_state = init != nullptr && slot >= 0;
    // channel j of the row `back` tokens before t as this sequence sees it: its own rows, else its
    // saved state, else 0
    auto tap = [&](int back, int j) -> float {
      if (t - back >= s0) return win[(rl - back) % K][j];
      if (from_state) return to_f32(init[slot * state_ss + (int64_t)(ch + j) * (K - 1) + (K - 1) - (s0 - (t - back))]);
      return 0.f;
    };
    float y[8];
    if (t - (K - 1) >= s0) {                                     // the common case: all taps inside the sequence
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        float acc = 0.f;
#pragma unroll
        for (int kk = 0; kk < K; ++kk) acc = fmaf(win[(rl - (K - 1) + kk) % K][j], wt[j][kk], acc);
        y[j] = x[j] + round_through<T>(acc);                     // x + conv(x), the conv rounded as eager does
      }
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        float acc = 0.f;
#pragma unroll
        for (int kk = 0; kk < K; ++kk) acc = fmaf(tap(K - 1 - kk, j), wt[j][kk], acc);
        y[j] = x[j] + round_through<T>(acc);
      }
    }
    store8<T>(dst + t * dst_row, y);
    if (cache != nullptr) {
      const int64_t cs = s_cs[i];
      if (cs >= 0) store8<T>(cache + cs * cache_row, y);
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

// ---- direct form (16-bit types, head_dim 128) -------------------------------------------------------------
// No tile shared between threads and no CTA-wide barrier.  A half warp (16 lanes x 8 channels = one head row of
// 128 channels) owns a stretch of consecutive groups of kDirTok tokens of one head; a warp is two head rows that
// are neighbours in memory, over the same tokens, so its control flow is the same in both halves and the row sums
// use full-mask shuffles of width 16.  The rows of the next group travel to a lane-private slot of shared memory
// while the current group is worked on (asynchronous 16-byte copies: in flight without holding registers).  Each
// row is normalised in registers, an fp32 window of K rows slides over the stretch (the K-1 rows at the end of a
// group are the next group's left context, so only the first group of a stretch reads halo rows), the arithmetic
// runs on channel pairs with the packed two-lane fp32 instructions, and q, k, v and the cache rows are written
// once.  Groups that touch a sequence start or end - two per sequence and head - take a per-token path that
// re-reads and re-normalises its taps.
constexpr int kDirTok = 8;                      // tokens per group (all loads of a group in flight together)
constexpr int kDirGroups = 4;                   // consecutive groups per half warp

template <typename T, int K>
__global__ void __launch_bounds__(128, 4)
qkv_prep_direct_kernel(const PrepArgs a, const int vec_weights, const int parts) {
  const int lane = threadIdx.x & 31;
  const int li = lane & 15;
  const int units = a.H + 2 * a.Hkv;
  const int n_groups = (a.total + kDirTok - 1) / kDirTok;
  // A warp = two head rows (neighbours in memory) over the same stretch of tokens, so its control flow is the same
  // in both halves and the row sums can use full-mask shuffles of width 16.  With an odd number of head rows the
  // last warp's second half shadows its partner: same loads and arithmetic, no stores.
  const int n_pairs = (units + 1) / 2;
  const int64_t wid = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  if (wid >= (int64_t)n_pairs * parts) return;                   // whole warps leave together
  const int u_raw = 2 * (int)(wid % n_pairs) + (lane >> 4);
  const bool active = u_raw < units;
  const int u = active ? u_raw : units - 1;
  const int part = (int)(wid / n_pairs);
  // this half warp's stretch of consecutive groups: the head row's groups cut into `parts` near-equal pieces
  const int g_begin = (int)((int64_t)part * n_groups / parts), g_end = (int)((int64_t)(part + 1) * n_groups / parts);
  const int which = u < a.H ? 0 : (u < a.H + a.Hkv ? 1 : 2);
  const int head = which == 0 ? u : (which == 1 ? u - a.H : u - a.H - a.Hkv);
  const int heads = which == 0 ? a.H : a.Hkv;
  const int dk = a.dk, c = li * 8, ch = head * dk + c;
  const T* src = which == 0 ? (const T*)a.qg + (int64_t)head * a.qg_head + c
                            : (which == 1 ? (const T*)a.k + head * dk + c : (const T*)a.v + head * dk + c);
  const int64_t row_st = which == 0 ? a.qg_row : (which == 1 ? a.k_row : a.v_row);
  const bool normalize = which != 2;
  const float inv_dk = 1.0f / (float)dk;
  T* dst = (T*)(which == 0 ? a.q_out : (which == 1 ? a.k_out : a.v_out)) + head * dk + c;
  T* cache = (which == 0 || a.k_cache == nullptr || !active) ? nullptr : (T*)(which == 1 ? a.k_cache : a.v_cache) + head * dk + c;
  const int64_t dst_row = (int64_t)heads * dk, cache_row = (int64_t)a.Hkv * dk;
  T* state = active ? (T*)a.state[which] : nullptr;
  const T* init = (const T*)a.init[which];
  const int64_t state_ss = a.state_ss[which];

  float2 wt2[4][K];                                               // the taps of channel pairs (2j, 2j+1)
  {
    float wt[8][K];
    const T* w = (const T*)a.w[which] + (int64_t)ch * K;
    if (vec_weights) {
      union { uint4 u4[K]; T e[8 * K]; } wv;
#pragma unroll
      for (int i = 0; i < K; ++i) wv.u4[i] = *reinterpret_cast<const uint4*>(w + i * 8);
#pragma unroll
      for (int j = 0; j < 8; ++j)
#pragma unroll
        for (int kk = 0; kk < K; ++kk) wt[j][kk] = to_f32(wv.e[j * K + kk]);
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j)
#pragma unroll
        for (int kk = 0; kk < K; ++kk) wt[j][kk] = to_f32(w[j * K + kk]);
    }
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int kk = 0; kk < K; ++kk) wt2[j][kk] = make_float2(wt[2 * j][kk], wt[2 * j + 1][kk]);
  }
  // normalise one row held as eight fp32 values.  v passes through the same instructions with a scale of one:
  // x * 1 and the rounding of a value that came from T leave it as it was, and the warp stays converged.
  auto norm_row = [&](float (&x)[8]) {
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) ss = fmaf(x[j], x[j], ss);
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o, 16);
    const float rs = normalize ? rsqrtf(ss * inv_dk + a.eps) : 1.0f;
#pragma unroll
    for (int j = 0; j < 8; ++j) x[j] *= rs;
    round8<T>(x);                                                // the eager op rounds to T here
  };

  // The half warp walks kDirGroups consecutive groups of kDirTok tokens.  After a group that lay inside one sequence
  // the last K-1 normalised rows are still in registers and serve as the next group's left context, so only the
  // first such group of a stretch pays for its halo rows.
  auto norm_row2 = [&](float2 (&x)[4]) {                          // norm_row on channel pairs, same summation order
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < 4; ++j) ss = fmaf(x[j].y, x[j].y, fmaf(x[j].x, x[j].x, ss));
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o, 16);
    const float rs = normalize ? rsqrtf(ss * inv_dk + a.eps) : 1.0f;
    const float2 rs2 = make_float2(rs, rs);
#pragma unroll
    for (int j = 0; j < 4; ++j) x[j] = __fmul2_rn(x[j], rs2);
    round8<T>(x);
  };
  float2 prevw[K - 1][4];                                         // the K-1 conv inputs before the next row, oldest first
  bool have_prev = false;
  // The rows of the next group travel to a lane-private slot of shared memory while this group is worked on
  // (asynchronous 16-byte copies: in flight without holding registers).  A lane reads back only what it copied
  // itself, so waiting for its own copy group is all the synchronisation there is.
  __shared__ uint4 s_next[2][kDirTok][128];
  auto request_group = [&](int g) {
    const int tn = g * kDirTok;
    if (g < g_end) {
#pragma unroll
      for (int rl = 0; rl < kDirTok; ++rl)
        if (tn + rl < a.total)
          mma::cp_async16(mma::smem_u32(&s_next[g & 1][rl][threadIdx.x]), src + (int64_t)(tn + rl) * row_st, true);
    }
    mma::cp_async_commit();
  };
  request_group(g_begin);
#pragma unroll 1
  for (int gi = g_begin; gi < g_end; ++gi) {
  const int t0 = gi * kDirTok;
  request_group(gi + 1);
  const int nt = min(kDirTok, a.total - t0);
  const int sa = a.seq_start[t0], sl = a.seq_start[t0 + nt - 1], ea = a.seq_end[t0 + nt - 1];
  const bool plain = nt == kDirTok && sa == sl && ea > t0 + nt && sa <= t0 - (K - 1);
  if (plain) {
    if (!have_prev) {
#pragma unroll
      for (int kk = 0; kk < K - 1; ++kk) {
        unpack8<T>(*reinterpret_cast<const uint4*>(src + (int64_t)(t0 - (K - 1) + kk) * row_st), prevw[kk]);
        norm_row2(prevw[kk]);
      }
    }
    mma::cp_async_wait<1>();                                       // this group's rows have landed (the next may be in flight)
#pragma unroll
    for (int rl = 0; rl < kDirTok; ++rl) {
      float2 x[4], y[4];
      unpack8<T>(s_next[gi & 1][rl][threadIdx.x], x);
      norm_row2(x);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float2 acc = make_float2(0.f, 0.f);
#pragma unroll
        for (int kk = 0; kk < K - 1; ++kk) acc = __ffma2_rn(prevw[kk][j], wt2[j][kk], acc);
        y[j] = __ffma2_rn(x[j], wt2[j][K - 1], acc);
      }
      round8<T>(y);                                              // the conv rounded as eager does, then x + conv(x)
#pragma unroll
      for (int j = 0; j < 4; ++j) y[j] = __fadd2_rn(y[j], x[j]);
      if (active) store8<T>(dst + (int64_t)(t0 + rl) * dst_row, y);
      if (cache != nullptr) {
        const long long cs = a.slot_mapping[t0 + rl];
        if (cs >= 0) store8<T>(cache + cs * cache_row, y);
      }
#pragma unroll
      for (int kk = 0; kk + 1 < K - 1; ++kk)
#pragma unroll
        for (int j = 0; j < 4; ++j) prevw[kk][j] = prevw[kk + 1][j];
#pragma unroll
      for (int j = 0; j < 4; ++j) prevw[K - 2][j] = x[j];
    }
    have_prev = true;
    continue;
  }
  have_prev = false;
  // ---- runs that touch a sequence border: token by token, tap by tap ---------------------------------------------
#pragma unroll 1
  for (int i = 0; i < kDirTok; ++i) {
    const int t = t0 + i;
    const bool t_on = t < a.total;                               // the same for the sixteen lanes
    const int tc = t_on ? t : 0;
    const int s0 = a.seq_start[tc], e0 = a.seq_end[tc], slot = a.seq_slot[tc];
    const bool from_state = init != nullptr && slot >= 0;
    float acc[8], cur[8], keep[K][8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
#pragma unroll
    for (int kk = 0; kk < K; ++kk) {
      const int back = K - 1 - kk, srow = tc - back;
      float x[8];
      load8<T>(src + (int64_t)max(srow, 0) * row_st, x);         // clamped; replaced below when before the start
      norm_row(x);
      if (srow < s0) {                                           // before the sequence start: saved state or zero
#pragma unroll
        for (int j = 0; j < 8; ++j)
          x[j] = from_state ? to_f32(init[slot * state_ss + (int64_t)(ch + j) * (K - 1) + (K - 1) - (s0 - srow)]) : 0.f;
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        acc[j] = fmaf(x[j], (j & 1) ? wt2[j >> 1][kk].y : wt2[j >> 1][kk].x, acc[j]);
        keep[kk][j] = x[j];
      }
      if (kk == K - 1) {
#pragma unroll
        for (int j = 0; j < 8; ++j) cur[j] = x[j];
      }
    }
    if (!t_on) continue;
    round8<T>(acc);
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] += cur[j];
    if (active) store8<T>(dst + (int64_t)t * dst_row, acc);
    if (cache != nullptr) {
      const long long cs = a.slot_mapping[t];
      if (cs >= 0) store8<T>(cache + cs * cache_row, acc);
    }
    if (t == e0 - 1 && state != nullptr && slot >= 0) {          // closes its sequence: its last K-1 conv inputs, oldest first
#pragma unroll
      for (int j = 0; j < 8; ++j)
#pragma unroll
        for (int kk = 0; kk < K - 1; ++kk)
          state[slot * state_ss + (int64_t)(ch + j) * (K - 1) + kk] = from_f32<T>(keep[kk + 1][j]);
    }
  }
  }                                                              // next group of the half warp
  mma::cp_async_wait<0>();
}

template <typename T>
int launch_prep(const PrepArgs& a, cudaStream_t st) {
  if constexpr (sizeof(T) == 2) {
    if (a.dk == 128) {                                           // the direct form: no shared-memory tile
      // every head row's groups are cut into stretches of about kDirGroups consecutive groups, one per half warp
      const int units = a.H + 2 * a.Hkv;
      const int n_groups = (a.total + kDirTok - 1) / kDirTok;
      const int parts = std::max(1, (n_groups + kDirGroups - 1) / kDirGroups);
      const int64_t warps = (int64_t)((units + 1) / 2) * parts;  // two head rows per warp
      const dim3 dgrid((unsigned)((warps + 3) / 4)), dblock(128);
      const int vec_w = ((reinterpret_cast<uintptr_t>(a.w[0]) | reinterpret_cast<uintptr_t>(a.w[1]) |
                          reinterpret_cast<uintptr_t>(a.w[2])) & 15) == 0 ? 1 : 0;
      switch (a.K) {
        case 2: qkv_prep_direct_kernel<T, 2><<<dgrid, dblock, 0, st>>>(a, vec_w, parts); break;
        case 3: qkv_prep_direct_kernel<T, 3><<<dgrid, dblock, 0, st>>>(a, vec_w, parts); break;
        default: qkv_prep_direct_kernel<T, 4><<<dgrid, dblock, 0, st>>>(a, vec_w, parts); break;
      }
      return launch_status("qkv_prep_prefill");
    }
  }
  const int smem = (kPrepTok + a.K - 1) * kPrepHeads * a.dk * (int)sizeof(T);
  dim3 grid((a.total + kPrepTok - 1) / kPrepTok, a.nq + (2 * a.Hkv + kPrepHeads - 1) / kPrepHeads), block(kPrepThreads);
#define ATMA_PREP_CASE(KK)                                                                                 \
  case KK: {                                                                                               \
    auto kern = qkv_prep_kernel<T, KK>;                                                                    \
    ATMA_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));           \
    kern<<<grid, block, smem, st>>>(a);                                                                    \
  } break;
  switch (a.K) { ATMA_PREP_CASE(2) ATMA_PREP_CASE(3) ATMA_PREP_CASE(4) }
#undef ATMA_PREP_CASE
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
  if (total <= 0) return ATMA_OK;
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
  a.nq = (H + kPrepHeads - 1) / kPrepHeads;
  int rc = ATMA_OK;
  ATMA_DISPATCH_DTYPE(dtype, T, { rc = launch_prep<T>(a, (cudaStream_t)stream); });
  return rc;
}
