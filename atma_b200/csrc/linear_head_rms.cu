// Projection + affine-free per-head RMSNorm (the reference keeps this as a prototype that is
// not on the model's path; it is provided for signature completeness).
// CTA = 16 rows x one head (width = head_dim or 2*head_dim columns); K is streamed through
// shared memory in slabs of 32; accumulation, the RMS statistic and the scaling are fp32.
#include "common.cuh"

namespace atma {

constexpr int kLhrRows = 16;
constexpr int kLhrSlab = 32;

template <typename T>
__global__ void __launch_bounds__(256)
linear_head_rms_kernel(const T* __restrict__ x, const T* __restrict__ w, const T* __restrict__ bias,
                       T* __restrict__ out, int M, int K, int heads, int head_dim, int width, float eps) {
  extern __shared__ float sm[];
  float* xs = sm;                                   // [16][33]
  float* ws = xs + kLhrRows * (kLhrSlab + 1);       // [width][33]
  float* os = ws + width * (kLhrSlab + 1);          // [16][width]
  __shared__ float s_rstd[kLhrRows];
  const int tid = threadIdx.x;
  const int m0 = blockIdx.x * kLhrRows, head = blockIdx.y;
  const int n_base = head * width;
  const int col = tid % width;                      // width is 128 or 256
  const int rgrp = tid / width;                     // 0 (width 256) or 0..1 (width 128)
  const int rows_per_thread = kLhrRows / (256 / width);
  float acc[kLhrRows];
#pragma unroll
  for (int i = 0; i < kLhrRows; ++i) acc[i] = 0.f;

  for (int k0 = 0; k0 < K; k0 += kLhrSlab) {
    for (int i = tid; i < kLhrRows * kLhrSlab; i += 256) {
      const int r = i / kLhrSlab, kk = i - r * kLhrSlab;
      xs[r * (kLhrSlab + 1) + kk] = (m0 + r < M && k0 + kk < K) ? to_f32(x[(int64_t)(m0 + r) * K + k0 + kk]) : 0.f;
    }
    for (int i = tid; i < width * kLhrSlab; i += 256) {
      const int n = i / kLhrSlab, kk = i - n * kLhrSlab;
      ws[n * (kLhrSlab + 1) + kk] = (k0 + kk < K) ? to_f32(w[(int64_t)(n_base + n) * K + k0 + kk]) : 0.f;
    }
    __syncthreads();
#pragma unroll 4
    for (int kk = 0; kk < kLhrSlab; ++kk) {
      const float wv = ws[col * (kLhrSlab + 1) + kk];
#pragma unroll
      for (int i = 0; i < kLhrRows; ++i)
        if (i < rows_per_thread) acc[i] = fmaf(xs[(rgrp * rows_per_thread + i) * (kLhrSlab + 1) + kk], wv, acc[i]);
    }
    __syncthreads();
  }
  const float bv = bias ? to_f32(bias[n_base + col]) : 0.f;
#pragma unroll
  for (int i = 0; i < kLhrRows; ++i)
    if (i < rows_per_thread) os[(rgrp * rows_per_thread + i) * width + col] = acc[i] + bv;
  __syncthreads();
  const int lane = tid & 31, warp = tid >> 5;
  for (int r = warp; r < kLhrRows; r += 8) {
    float s = 0.f;
    for (int d = lane; d < head_dim; d += 32) { const float t = os[r * width + d]; s = fmaf(t, t, s); }
    s = warp_sum(s);
    if (lane == 0) s_rstd[r] = rsqrtf(s / (float)head_dim + eps);
  }
  __syncthreads();
  for (int i = tid; i < kLhrRows * width; i += 256) {
    const int r = i / width, n = i - r * width;
    if (m0 + r < M) {
      const float t = os[i] * (n < head_dim ? s_rstd[r] : 1.0f);
      out[(int64_t)(m0 + r) * heads * width + n_base + n] = from_f32<T>(t);
    }
  }
}

}  // namespace atma

using namespace atma;

extern "C" int atma_linear_head_rms(const void* x, const void* weight, const void* bias, void* out,
                                    int M, int K, int heads, int head_dim, int gated, float eps,
                                    int dtype, void* stream) {
  ATMA_REQUIRE(dtype_ok(dtype), "linear_head_rms: unsupported dtype %d", dtype);
  ATMA_REQUIRE(head_dim == 128, "linear_head_rms: head_dim %d (only 128 is supported)", head_dim);
  if (M <= 0 || heads <= 0) return ATMA_OK;
  const int width = head_dim * (gated ? 2 : 1);
  const size_t smem = sizeof(float) * ((size_t)kLhrRows * (kLhrSlab + 1) + (size_t)width * (kLhrSlab + 1) +
                                       (size_t)kLhrRows * width);
  dim3 grid((M + kLhrRows - 1) / kLhrRows, heads);
  int rc = ATMA_OK;
  ATMA_DISPATCH_DTYPE(dtype, T, {
    auto kern = linear_head_rms_kernel<T>;
    ATMA_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    kern<<<grid, 256, smem, (cudaStream_t)stream>>>((const T*)x, (const T*)weight, (const T*)bias, (T*)out,
                                                    M, K, heads, head_dim, width, eps);
    rc = launch_status("linear_head_rms");
  });
  return rc;
}
