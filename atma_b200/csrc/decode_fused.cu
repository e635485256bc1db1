// Decode-side glue of a global layer and of the residual stream, one launch each.
//
// (1) qkv_prep_decode: what the reference's decode branch does between the q/k/v projections
//     and the attention kernel - per-head RMSNorm of q and k, the three depthwise "Canon" conv
//     steps in residual form with their slot-indexed state rows, and the scatter of the new K/V
//     row into the paged cache (inference/models/atma.py:552-572: two F.rms_norm, three
//     _gpu_conv_step, three adds, store_kvcache) - as ONE kernel: a warp owns one head of one
//     token, each lane dk/32 neighbouring channels, the row's mean square comes from one warp
//     reduction, every conv-state row is read and written once.
// (2) add_rms_norm: the residual add followed by the next RMSNorm (x <- x + y; h = norm(x) * w),
//     which the block structure x + attn(norm1(x)), x + mlp(norm2(x)) repeats twice per layer
//     (inference/models/atma.py:709-712; model/layers.py:14-17).
// Rounding follows eager execution: every op of the reference rounds its result to the
// activation dtype, and so do the corresponding points here.
#include "common.cuh"

namespace atma {

namespace {

constexpr int kMaxConvK = 4;

struct PrepDecodeArgs {
  const void* qg; int64_t qg_row, qg_head;       // q at the start of each head's [q | gate] chunk
  const void* k; int64_t k_row;
  const void* v; int64_t v_row;
  const void* w[3];                               // [C][K] conv weights of q, k, v
  void* state[3]; int64_t state_ss[3];            // [rows][C][K-1] conv-state tables, updated in place
  const int64_t* slots;                           // [B] state rows (negative: padded batch row)
  void* q_out; void* k_out; void* v_out;          // dense [B][heads][dk]
  void* k_cache; void* v_cache; const int32_t* slot_mapping;   // cache rows [slot][Hkv][dk]; -1 = skip
  int B, H, Hkv, dk, K;
  float eps;
};

// Loads of CPL consecutive 16-bit values as one access when CPL * 2 bytes is 8 or 16 (the lane's channels,
// their K taps and their K-1 state values are each contiguous), else element by element.
template <typename T, int N>
__device__ __forceinline__ void load_run(const T* p, T (&o)[N]) {
  if constexpr (N * sizeof(T) == 16) {
    *reinterpret_cast<uint4*>(o) = *reinterpret_cast<const uint4*>(p);
  } else if constexpr (N * sizeof(T) == 8) {
    *reinterpret_cast<uint2*>(o) = *reinterpret_cast<const uint2*>(p);
  } else if constexpr (N * sizeof(T) % 8 == 0) {
#pragma unroll
    for (int i = 0; i < (int)(N * sizeof(T) / 8); ++i) reinterpret_cast<uint2*>(o)[i] = reinterpret_cast<const uint2*>(p)[i];
  } else {
#pragma unroll
    for (int i = 0; i < N; ++i) o[i] = p[i];
  }
}
template <typename T, int N>
__device__ __forceinline__ void store_run(T* p, const T (&v)[N]) {
  if constexpr (N * sizeof(T) == 16) {
    *reinterpret_cast<uint4*>(p) = *reinterpret_cast<const uint4*>(v);
  } else if constexpr (N * sizeof(T) == 8) {
    *reinterpret_cast<uint2*>(p) = *reinterpret_cast<const uint2*>(v);
  } else if constexpr (N * sizeof(T) % 8 == 0) {
#pragma unroll
    for (int i = 0; i < (int)(N * sizeof(T) / 8); ++i) reinterpret_cast<uint2*>(p)[i] = reinterpret_cast<const uint2*>(v)[i];
  } else {
#pragma unroll
    for (int i = 0; i < N; ++i) p[i] = v[i];
  }
}

// K is a template parameter so that the lane's K taps and K-1 state values per channel form compile-time runs:
// everything the lane needs (its channels of the token row, their taps, their state) is requested up front in a
// handful of wide loads, then normalised, convolved and written.  `wide`: pointers and strides allow the wide form.
template <typename T, int CPL, int K>
__global__ void __launch_bounds__(128)
qkv_prep_decode_kernel(const PrepDecodeArgs a, const int wide) {
  const int lane = threadIdx.x & 31;
  const int unit = blockIdx.x * 4 + (threadIdx.x >> 5);
  const int units = a.H + 2 * a.Hkv;
  if (unit >= a.B * units) return;
  const int b = unit / units, u = unit % units;
  const int which = u < a.H ? 0 : (u < a.H + a.Hkv ? 1 : 2);      // q, k, v
  const int head = which == 0 ? u : (which == 1 ? u - a.H : u - a.H - a.Hkv);
  const int heads = which == 0 ? a.H : a.Hkv;
  const T* src = which == 0 ? static_cast<const T*>(a.qg) + b * a.qg_row + head * a.qg_head
                            : (which == 1 ? static_cast<const T*>(a.k) + b * a.k_row + head * a.dk
                                          : static_cast<const T*>(a.v) + b * a.v_row + head * a.dk);
  const int c0 = lane * CPL;                                      // channel inside the head
  const int64_t slot = a.slots[b];
  const T* wp = static_cast<const T*>(a.w[which]) + (int64_t)(head * a.dk + c0) * K;
  T* st = slot >= 0 ? static_cast<T*>(a.state[which]) + slot * a.state_ss[which] + (int64_t)(head * a.dk + c0) * (K - 1) : nullptr;
  T xr[CPL], wr[CPL * K], sr[CPL * (K - 1)];
  if (wide) {
    load_run<T, CPL>(src + c0, xr);
    load_run<T, CPL * K>(wp, wr);
    if (st != nullptr) load_run<T, CPL * (K - 1)>(st, sr);
  } else {
#pragma unroll
    for (int j = 0; j < CPL; ++j) xr[j] = src[c0 + j];
#pragma unroll
    for (int j = 0; j < CPL * K; ++j) wr[j] = wp[j];
    if (st != nullptr) {
#pragma unroll
      for (int j = 0; j < CPL * (K - 1); ++j) sr[j] = st[j];
    }
  }
  float x[CPL];
#pragma unroll
  for (int j = 0; j < CPL; ++j) x[j] = to_f32(xr[j]);
  if (which != 2) {                                               // per-head RMSNorm of q and k (affine-free)
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < CPL; ++j) ss = fmaf(x[j], x[j], ss);
    ss = warp_sum(ss);
    const float rs = rsqrtf(ss / (float)a.dk + a.eps);
#pragma unroll
    for (int j = 0; j < CPL; ++j) x[j] = round_through<T>(x[j] * rs);
  }
  T yo[CPL], sn[CPL * (K - 1)];
#pragma unroll
  for (int j = 0; j < CPL; ++j) {
    float acc = x[j] * to_f32(wr[j * K + K - 1]);
    if (st != nullptr) {
#pragma unroll
      for (int t = 0; t < K - 1; ++t) acc = fmaf(to_f32(sr[j * (K - 1) + t]), to_f32(wr[j * K + t]), acc);
#pragma unroll
      for (int t = 0; t + 1 < K - 1; ++t) sn[j * (K - 1) + t] = sr[j * (K - 1) + t + 1];
      sn[j * (K - 1) + K - 2] = from_f32<T>(x[j]);
    }
    yo[j] = from_f32<T>(x[j] + round_through<T>(acc));           // x + conv(x)
  }
  T* dst = (which == 0 ? static_cast<T*>(a.q_out) : (which == 1 ? static_cast<T*>(a.k_out) : static_cast<T*>(a.v_out))) +
           ((int64_t)b * heads + head) * a.dk + c0;
  T* cr = nullptr;
  if (which != 0 && a.k_cache != nullptr) {
    const int cs = a.slot_mapping[b];
    if (cs >= 0) cr = (which == 1 ? static_cast<T*>(a.k_cache) : static_cast<T*>(a.v_cache)) + ((int64_t)cs * a.Hkv + head) * a.dk + c0;
  }
  if (wide) {
    if (st != nullptr) store_run<T, CPL * (K - 1)>(st, sn);
    store_run<T, CPL>(dst, yo);
    if (cr != nullptr) store_run<T, CPL>(cr, yo);
  } else {
    if (st != nullptr) {
#pragma unroll
      for (int j = 0; j < CPL * (K - 1); ++j) st[j] = sn[j];
    }
#pragma unroll
    for (int j = 0; j < CPL; ++j) dst[j] = yo[j];
    if (cr != nullptr) {
#pragma unroll
      for (int j = 0; j < CPL; ++j) cr[j] = yo[j];
    }
  }
}

// x_out = x + y (rounded to T); h = x_out * rsqrt(mean(x_out^2) + eps) * w.  One warp per row when D <= 2048:
// lane holds D/32 values in registers between the two passes.
template <typename T, int VPL>
__global__ void __launch_bounds__(128)
add_rms_norm_kernel(const T* __restrict__ x, const T* __restrict__ y, const T* __restrict__ w, T* __restrict__ x_out,
                    T* __restrict__ h_out, int rows, int D, float eps) {
  const int lane = threadIdx.x & 31;
  const int row = blockIdx.x * 4 + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int64_t base = (int64_t)row * D;
  float v[VPL];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < VPL; ++i) {
    const int c = (i * 32 + lane);                               // interleaved: neighbouring lanes, neighbouring addresses
    float t = c < D ? to_f32(x[base + c]) : 0.f;
    if (y != nullptr && c < D) t = round_through<T>(t + to_f32(y[base + c]));
    v[i] = t;
    ss = fmaf(t, t, ss);
  }
  ss = warp_sum(ss);
  const float rs = rsqrtf(ss / (float)D + eps);
#pragma unroll
  for (int i = 0; i < VPL; ++i) {
    const int c = i * 32 + lane;
    if (c < D) {
      if (x_out != nullptr) x_out[base + c] = from_f32<T>(v[i]);
      h_out[base + c] = from_f32<T>(v[i] * rs * (w != nullptr ? to_f32(w[c]) : 1.f));
    }
  }
}

// The same for rows whose length is a multiple of eight 16-bit values (16-byte aligned): one CTA per row, one
// 16-byte piece per thread, so that a row is one round of loads, a block reduction and one round of stores -
// the latency of a decode step's 2 x layers launches of this kernel, not its bandwidth, is what counts.
template <typename T>
__global__ void __launch_bounds__(512)
add_rms_norm_row_kernel(const T* __restrict__ x, const T* __restrict__ y, const T* __restrict__ w, T* __restrict__ x_out,
                        T* __restrict__ h_out, int D, float eps) {
  __shared__ float s_part[16];
  const int row = blockIdx.x, tid = threadIdx.x;
  const int c = tid * 8;
  const bool on = c < D;
  const int64_t base = (int64_t)row * D + c;
  union V8 { uint4 u; T e[8]; };
  V8 xv, yv, wv;
  xv.u = on ? *reinterpret_cast<const uint4*>(x + base) : make_uint4(0u, 0u, 0u, 0u);
  if (y != nullptr) yv.u = on ? *reinterpret_cast<const uint4*>(y + base) : make_uint4(0u, 0u, 0u, 0u);
  if (w != nullptr) wv.u = on ? *reinterpret_cast<const uint4*>(w + c) : make_uint4(0u, 0u, 0u, 0u);
  float v[8];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    float t = to_f32(xv.e[i]);
    if (y != nullptr) t = round_through<T>(t + to_f32(yv.e[i]));
    v[i] = t;
    ss = fmaf(t, t, ss);
  }
  ss = warp_sum(ss);
  if ((tid & 31) == 0) s_part[tid >> 5] = ss;
  __syncthreads();
  float tot = 0.f;
  for (int i = 0; i < (int)(blockDim.x >> 5); ++i) tot += s_part[i];
  const float rs = rsqrtf(tot / (float)D + eps);
  if (!on) return;
  V8 xo, ho;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    xo.e[i] = from_f32<T>(v[i]);
    ho.e[i] = from_f32<T>(v[i] * rs * (w != nullptr ? to_f32(wv.e[i]) : 1.f));
  }
  if (x_out != nullptr) *reinterpret_cast<uint4*>(x_out + base) = xo.u;
  *reinterpret_cast<uint4*>(h_out + base) = ho.u;
}

}  // namespace
}  // namespace atma

using namespace atma;

extern "C" int atma_qkv_prep_decode(const void* q_gate, int64_t qg_row, int64_t qg_head, const void* k, int64_t k_row,
                                    const void* v, int64_t v_row, const void* w_q, const void* w_k, const void* w_v,
                                    void* state_q, void* state_k, void* state_v, int64_t ss_q, int64_t ss_k, int64_t ss_v,
                                    const int64_t* slots, void* q_out, void* k_out, void* v_out, void* k_cache,
                                    void* v_cache, const int32_t* slot_mapping, int B, int H, int Hkv, int dk, int K,
                                    float eps, int dtype, void* stream) {
  ATMA_REQUIRE(dtype_ok(dtype), "qkv_prep_decode: unsupported dtype %d", dtype);
  ATMA_REQUIRE(dk == 32 || dk == 64 || dk == 128 || dk == 256, "qkv_prep_decode: head_dim %d not in {32,64,128,256}", dk);
  ATMA_REQUIRE(K >= 2 && K <= kMaxConvK, "qkv_prep_decode: kernel size %d not in 2..%d", K, kMaxConvK);
  ATMA_REQUIRE(H > 0 && Hkv > 0 && H % Hkv == 0, "qkv_prep_decode: bad head counts");
  ATMA_REQUIRE(slots != nullptr && state_q != nullptr && state_k != nullptr && state_v != nullptr,
               "qkv_prep_decode: the three conv-state tables and the slot list are required");
  ATMA_REQUIRE(k_cache == nullptr || (v_cache != nullptr && slot_mapping != nullptr), "qkv_prep_decode: caches need a slot mapping");
  if (B <= 0) return ATMA_OK;
  PrepDecodeArgs a{};
  a.qg = q_gate; a.qg_row = qg_row; a.qg_head = qg_head; a.k = k; a.k_row = k_row; a.v = v; a.v_row = v_row;
  a.w[0] = w_q; a.w[1] = w_k; a.w[2] = w_v;
  a.state[0] = state_q; a.state[1] = state_k; a.state[2] = state_v;
  a.state_ss[0] = ss_q; a.state_ss[1] = ss_k; a.state_ss[2] = ss_v;
  a.slots = slots; a.q_out = q_out; a.k_out = k_out; a.v_out = v_out;
  a.k_cache = k_cache; a.v_cache = v_cache; a.slot_mapping = slot_mapping;
  a.B = B; a.H = H; a.Hkv = Hkv; a.dk = dk; a.K = K; a.eps = eps;
  const int units = B * (H + 2 * Hkv);
  const dim3 grid((units + 3) / 4), block(128);
  cudaStream_t st = (cudaStream_t)stream;
  // the wide form needs aligned runs: CPL * 2 bytes per lane of every row, CPL * K * 2 of taps, CPL * (K-1) * 2 of state
  auto al = [](const void* p, int n) { return (reinterpret_cast<uintptr_t>(p) & (uintptr_t)(n - 1)) == 0; };
  const bool two_byte = dtype != ATMA_F32;
  const int wide = (two_byte && (dk == 128 || dk == 256) && qg_row % 8 == 0 && qg_head % 8 == 0 && k_row % 8 == 0 && v_row % 8 == 0 &&
                    ss_q % 8 == 0 && ss_k % 8 == 0 && ss_v % 8 == 0 && al(q_gate, 16) && al(k, 16) && al(v, 16) && al(w_q, 16) &&
                    al(w_k, 16) && al(w_v, 16) && al(state_q, 16) && al(state_k, 16) && al(state_v, 16) && al(q_out, 16) &&
                    al(k_out, 16) && al(v_out, 16) && al(k_cache, 16) && al(v_cache, 16)) ? 1 : 0;
#define ATMA_PD(CPLV)                                                                        \
  switch (K) {                                                                               \
    case 2: qkv_prep_decode_kernel<T, CPLV, 2><<<grid, block, 0, st>>>(a, wide); break;      \
    case 3: qkv_prep_decode_kernel<T, CPLV, 3><<<grid, block, 0, st>>>(a, wide); break;      \
    default: qkv_prep_decode_kernel<T, CPLV, 4><<<grid, block, 0, st>>>(a, wide); break;     \
  }
  ATMA_DISPATCH_DTYPE(dtype, T, {
    switch (dk) {
      case 32: ATMA_PD(1) break;
      case 64: ATMA_PD(2) break;
      case 128: ATMA_PD(4) break;
      default: ATMA_PD(8) break;
    }
  });
#undef ATMA_PD
  return launch_status("qkv_prep_decode");
}

extern "C" int atma_add_rms_norm(const void* x, const void* y, const void* weight, void* x_out, void* h_out, int rows, int D,
                                 float eps, int dtype, void* stream) {
  ATMA_REQUIRE(dtype_ok(dtype), "add_rms_norm: unsupported dtype %d", dtype);
  ATMA_REQUIRE(D >= 1 && D <= 4096, "add_rms_norm: D=%d outside 1..4096", D);
  ATMA_REQUIRE(x != nullptr && h_out != nullptr, "add_rms_norm: x and h_out are required");
  if (rows <= 0) return ATMA_OK;
  cudaStream_t st = (cudaStream_t)stream;
  auto al16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
  if (dtype != ATMA_F32 && D % 8 == 0 && al16(x) && al16(y) && al16(weight) && al16(x_out) && al16(h_out)) {
    const int threads = ((D / 8 + 31) / 32) * 32;                // <= 512 for D <= 4096
    if (dtype == ATMA_BF16)
      add_rms_norm_row_kernel<__nv_bfloat16><<<rows, threads, 0, st>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)y,
          (const __nv_bfloat16*)weight, (__nv_bfloat16*)x_out, (__nv_bfloat16*)h_out, D, eps);
    else
      add_rms_norm_row_kernel<__half><<<rows, threads, 0, st>>>((const __half*)x, (const __half*)y, (const __half*)weight,
                                                                (__half*)x_out, (__half*)h_out, D, eps);
    return launch_status("add_rms_norm");
  }
  const dim3 grid((rows + 3) / 4), block(128);
  const int vpl = (D + 31) / 32;
  ATMA_DISPATCH_DTYPE(dtype, T, {
    const T* xp = (const T*)x; const T* yp = (const T*)y; const T* wp = (const T*)weight;
    T* xo = (T*)x_out; T* ho = (T*)h_out;
    if (vpl <= 8) add_rms_norm_kernel<T, 8><<<grid, block, 0, st>>>(xp, yp, wp, xo, ho, rows, D, eps);
    else if (vpl <= 32) add_rms_norm_kernel<T, 32><<<grid, block, 0, st>>>(xp, yp, wp, xo, ho, rows, D, eps);
    else if (vpl <= 64) add_rms_norm_kernel<T, 64><<<grid, block, 0, st>>>(xp, yp, wp, xo, ho, rows, D, eps);
    else add_rms_norm_kernel<T, 128><<<grid, block, 0, st>>>(xp, yp, wp, xo, ho, rows, D, eps);
  });
  return launch_status("add_rms_norm");
}
