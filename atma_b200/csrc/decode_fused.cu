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

template <typename T, int CPL>
__global__ void __launch_bounds__(128)
qkv_prep_decode_kernel(const PrepDecodeArgs a) {
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
  float x[CPL];
#pragma unroll
  for (int j = 0; j < CPL; ++j) x[j] = to_f32(src[c0 + j]);
  if (which != 2) {                                               // per-head RMSNorm of q and k (affine-free)
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < CPL; ++j) ss = fmaf(x[j], x[j], ss);
    ss = warp_sum(ss);
    const float rs = rsqrtf(ss / (float)a.dk + a.eps);
#pragma unroll
    for (int j = 0; j < CPL; ++j) x[j] = round_through<T>(x[j] * rs);
  }
  const int64_t slot = a.slots[b];
  const int K = a.K;
  const T* w = static_cast<const T*>(a.w[which]) + (int64_t)(head * a.dk + c0) * K;
  T* st = slot >= 0 ? static_cast<T*>(a.state[which]) + slot * a.state_ss[which] + (int64_t)(head * a.dk + c0) * (K - 1) : nullptr;
  float y[CPL];
#pragma unroll
  for (int j = 0; j < CPL; ++j) {
    float acc = x[j] * to_f32(w[j * K + K - 1]);
    if (st != nullptr) {
      T old[kMaxConvK - 1];
      for (int t = 0; t < K - 1; ++t) old[t] = st[j * (K - 1) + t];
      for (int t = 0; t < K - 1; ++t) acc = fmaf(to_f32(old[t]), to_f32(w[j * K + t]), acc);
      for (int t = 0; t + 1 < K - 1; ++t) st[j * (K - 1) + t] = old[t + 1];
      st[j * (K - 1) + K - 2] = from_f32<T>(x[j]);
    }
    y[j] = round_through<T>(x[j] + round_through<T>(acc));      // x + conv(x)
  }
  T* dst = (which == 0 ? static_cast<T*>(a.q_out) : (which == 1 ? static_cast<T*>(a.k_out) : static_cast<T*>(a.v_out))) +
           ((int64_t)b * heads + head) * a.dk + c0;
#pragma unroll
  for (int j = 0; j < CPL; ++j) dst[j] = from_f32<T>(y[j]);
  if (which != 0 && a.k_cache != nullptr) {
    const int cs = a.slot_mapping[b];
    if (cs >= 0) {
      T* cr = (which == 1 ? static_cast<T*>(a.k_cache) : static_cast<T*>(a.v_cache)) + ((int64_t)cs * a.Hkv + head) * a.dk + c0;
#pragma unroll
      for (int j = 0; j < CPL; ++j) cr[j] = from_f32<T>(y[j]);
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
  ATMA_DISPATCH_DTYPE(dtype, T, {
    switch (dk) {
      case 32: qkv_prep_decode_kernel<T, 1><<<grid, block, 0, st>>>(a); break;
      case 64: qkv_prep_decode_kernel<T, 2><<<grid, block, 0, st>>>(a); break;
      case 128: qkv_prep_decode_kernel<T, 4><<<grid, block, 0, st>>>(a); break;
      default: qkv_prep_decode_kernel<T, 8><<<grid, block, 0, st>>>(a); break;
    }
  });
  return launch_status("qkv_prep_decode");
}

extern "C" int atma_add_rms_norm(const void* x, const void* y, const void* weight, void* x_out, void* h_out, int rows, int D,
                                 float eps, int dtype, void* stream) {
  ATMA_REQUIRE(dtype_ok(dtype), "add_rms_norm: unsupported dtype %d", dtype);
  ATMA_REQUIRE(D >= 1 && D <= 4096, "add_rms_norm: D=%d outside 1..4096", D);
  ATMA_REQUIRE(x != nullptr && h_out != nullptr, "add_rms_norm: x and h_out are required");
  if (rows <= 0) return ATMA_OK;
  const dim3 grid((rows + 3) / 4), block(128);
  cudaStream_t st = (cudaStream_t)stream;
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
