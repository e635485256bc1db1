// Weight-streaming linear layers for small decode batches (up to 16 rows): out = x W^T + b, optionally
// with the MLP's squared-ReLU gate applied to the two halves of the result before it is written
// (inference/models/atma.py:87-97: fc GEMM -> gate * relu(x)^2 -> proj GEMM; :631-673: in_proj / out_proj
// around the LFM2 conv).  At these batch sizes the products are bound by reading the weights once from
// HBM: every warp streams whole 16-row slabs of W with 16-byte loads (all loads of its K range in flight
// before the first use), keeps them in the register layout mma.sync wants without a shared-memory round
// trip, and multiplies by the x rows it reads from L1/L2.  A 16-byte piece of a weight row is eight
// consecutive k; the same eight k of an x row go to the matching B-operand registers, so the reduction
// index is permuted identically on both sides and no shuffle is needed.  K is split over the 16 warps of a
// CTA; their partial tiles meet in shared memory, where bias, rounding to the activation dtype (what the
// GEMM of the separate-op path would have written) and the gate are applied.
#include "common.cuh"
#include "mma_sync.cuh"

namespace atma {

namespace {

constexpr int kWarps = 16;                 // warps per CTA
constexpr int kMaxRows = 16;               // batch rows (two n8 tiles)

struct LinArgs {
  const void* x; int64_t x_rs;             // [B][K]
  const void* w;                           // [N][K] row-major (torch Linear layout)
  const void* bias;                        // [N] or null
  void* out; int64_t out_rs;               // [B][N] (plain) or [B][N/2] (gated)
  int B, N, K;
  int ks;                                  // K splits per unit (power of two <= 16); units per CTA = 16 / ks
  int units;                               // 16-feature units (gated: N/2/16, else N/16)
};

// One warp: its unit's rows [row0, row0+16) (and, gated, [row0 + N/2, ...)) over k in [k0, k1).
template <typename T, int NT, bool kGated>
__global__ void __launch_bounds__(kWarps * 32)
decode_linear_kernel(const LinArgs a) {
  constexpr bool kBf16 = std::is_same<T, __nv_bfloat16>::value;
  constexpr int kTiles = kGated ? 2 : 1;
  __shared__ float part[kWarps][kTiles][NT][4][32];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int upc = kWarps / a.ks;                              // units per CTA
  const int unit = blockIdx.x * upc + warp / a.ks;
  const int split = warp % a.ks;
  const int kper = a.K / a.ks;                                // multiple of 32 (checked on the host)
  const int k0 = split * kper;
  const T* W = static_cast<const T*>(a.w);
  const T* X = static_cast<const T*>(a.x);
  float acc[kTiles][NT][4];
#pragma unroll
  for (int i = 0; i < kTiles; ++i)
#pragma unroll
    for (int n = 0; n < NT; ++n)
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[i][n][j] = 0.f;

  if (unit < a.units) {
    const int row0 = unit * 16;
    const T* wr[kTiles][2];
#pragma unroll
    for (int i = 0; i < kTiles; ++i) {
      const int64_t base = (int64_t)(row0 + (i ? a.N / 2 : 0));
      wr[i][0] = W + (base + g) * a.K + k0 + 8 * t;
      wr[i][1] = W + (base + g + 8) * a.K + k0 + 8 * t;
    }
    const T* xr[NT];
    bool xok[NT];
#pragma unroll
    for (int n = 0; n < NT; ++n) {
      xok[n] = (8 * n + g) < a.B;
      xr[n] = X + (int64_t)(xok[n] ? 8 * n + g : 0) * a.x_rs + k0 + 8 * t;
    }
    constexpr int kUnroll = 4;                                // 32-k blocks requested together
    for (int kb = 0; kb < kper; kb += 32 * kUnroll) {
      uint4 wv[kUnroll][kTiles][2], xv[kUnroll][NT];
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        const bool on = kb + 32 * u < kper;
#pragma unroll
        for (int i = 0; i < kTiles; ++i)
#pragma unroll
          for (int r = 0; r < 2; ++r)
            wv[u][i][r] = on ? __ldcs(reinterpret_cast<const uint4*>(wr[i][r] + kb + 32 * u)) : make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
        for (int n = 0; n < NT; ++n)
          xv[u][n] = (on && xok[n]) ? *reinterpret_cast<const uint4*>(xr[n] + kb + 32 * u) : make_uint4(0u, 0u, 0u, 0u);
      }
#pragma unroll
      for (int u = 0; u < kUnroll; ++u)
#pragma unroll
        for (int i = 0; i < kTiles; ++i)
#pragma unroll
          for (int n = 0; n < NT; ++n) {
            const uint32_t a0[4] = {wv[u][i][0].x, wv[u][i][1].x, wv[u][i][0].y, wv[u][i][1].y};
            const uint32_t a1[4] = {wv[u][i][0].z, wv[u][i][1].z, wv[u][i][0].w, wv[u][i][1].w};
            mma::mma16816<kBf16>(acc[i][n], a0, xv[u][n].x, xv[u][n].y);
            mma::mma16816<kBf16>(acc[i][n], a1, xv[u][n].z, xv[u][n].w);
          }
    }
  }
#pragma unroll
  for (int i = 0; i < kTiles; ++i)
#pragma unroll
    for (int n = 0; n < NT; ++n)
#pragma unroll
      for (int j = 0; j < 4; ++j) part[warp][i][n][j][lane] = acc[i][n][j];
  __syncthreads();
  // the first warp of every unit adds the K splits and writes the unit's 16 features of every batch row
  if (split != 0 || unit >= a.units) return;
  const int row0 = unit * 16;
  const T* bias = static_cast<const T*>(a.bias);
  T* out = static_cast<T*>(a.out);
#pragma unroll
  for (int n = 0; n < NT; ++n) {
    float y[kTiles][4];
#pragma unroll
    for (int i = 0; i < kTiles; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float s = 0.f;
        for (int k = 0; k < a.ks; ++k) s += part[warp + k][i][n][j][lane];
        const int feat = row0 + (i ? a.N / 2 : 0) + g + (j >= 2 ? 8 : 0);
        if (bias != nullptr) s += to_f32(bias[feat]);
        y[i][j] = round_through<T>(s);                         // what the GEMM of the separate-op path writes
      }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int b = 8 * n + 2 * t + (j & 1);
      const int feat = row0 + g + (j >= 2 ? 8 : 0);
      if (b >= a.B) continue;
      float v = y[0][j];
      if constexpr (kGated) {
        const float p = fmaxf(y[0][j], 0.f);
        float sq = p * p;
        if constexpr (kBf16) sq = round_through<T>(sq);         // eager bf16 materialises relu(x)^2 before the multiply
        v = y[1][j] * sq;
      }
      out[(int64_t)b * a.out_rs + feat] = from_f32<T>(v);
    }
  }
}

}  // namespace
}  // namespace atma

using namespace atma;

extern "C" int atma_decode_linear(const void* x, int64_t x_row_stride, const void* weight, const void* bias, void* out,
                                  int64_t out_row_stride, int B, int N, int K, int gated, int dtype, void* stream) {
  ATMA_REQUIRE(dtype == ATMA_BF16 || dtype == ATMA_F16, "decode_linear: 16-bit activations and weights only (dtype %d)", dtype);
  ATMA_REQUIRE(B >= 0 && B <= kMaxRows, "decode_linear: %d rows; this entry serves decode batches of up to %d", B, kMaxRows);
  ATMA_REQUIRE(K >= 32 && K % 32 == 0, "decode_linear: K=%d must be a multiple of 32", K);
  ATMA_REQUIRE(N > 0 && N % (gated ? 32 : 16) == 0, "decode_linear: N=%d must be a multiple of %d", N, gated ? 32 : 16);
  ATMA_REQUIRE((reinterpret_cast<uintptr_t>(x) & 15) == 0 && (reinterpret_cast<uintptr_t>(weight) & 15) == 0 && x_row_stride % 8 == 0,
               "decode_linear: x and weight must be 16-byte aligned with a row stride that is a multiple of 8 elements");
  if (B == 0) return ATMA_OK;
  LinArgs a{};
  a.x = x; a.x_rs = x_row_stride; a.w = weight; a.bias = bias; a.out = out; a.out_rs = out_row_stride;
  a.B = B; a.N = N; a.K = K;
  a.units = (gated ? N / 2 : N) / 16;
  // K splits per unit: as many as give every split whole 32-k blocks and keep the grid within one wave
  const int sms = sm_count_of_current_device();
  int ks = kWarps;
  while (ks > 1 && (K % (32 * ks) != 0 || (int64_t)a.units * ks / kWarps > sms)) ks >>= 1;
  a.ks = ks;
  const int upc = kWarps / ks;
  const dim3 grid((a.units + upc - 1) / upc), block(kWarps * 32);
  cudaStream_t st = (cudaStream_t)stream;
#define ATMA_LIN(T, NT, G) decode_linear_kernel<T, NT, G><<<grid, block, 0, st>>>(a)
  if (dtype == ATMA_BF16) {
    if (B <= 8) { if (gated) ATMA_LIN(__nv_bfloat16, 1, true); else ATMA_LIN(__nv_bfloat16, 1, false); }
    else { if (gated) ATMA_LIN(__nv_bfloat16, 2, true); else ATMA_LIN(__nv_bfloat16, 2, false); }
  } else {
    if (B <= 8) { if (gated) ATMA_LIN(__half, 1, true); else ATMA_LIN(__half, 1, false); }
    else { if (gated) ATMA_LIN(__half, 2, true); else ATMA_LIN(__half, 2, false); }
  }
#undef ATMA_LIN
  return launch_status("decode_linear");
}
