// Shared helpers for the C-ABI kernels: error reporting, dtype-generic loads/stores.
#pragma once

#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cstdint>
#include <cstdio>
#include <cstdarg>
#include <type_traits>

#include "../../include/atma_b200.h"

namespace atma {

// Thread-local message for the last failing call (read through atma_last_error()).
char* err_buf();
int fail(int code, const char* fmt, ...);

#define ATMA_REQUIRE(cond, ...)                                    \
  do {                                                             \
    if (!(cond)) return ::atma::fail(ATMA_ERR_INVALID, __VA_ARGS__); \
  } while (0)

#define ATMA_CUDA_OK(expr)                                                         \
  do {                                                                             \
    cudaError_t e__ = (expr);                                                      \
    if (e__ != cudaSuccess)                                                        \
      return ::atma::fail(ATMA_ERR_CUDA, "%s: %s", #expr, cudaGetErrorString(e__)); \
  } while (0)

inline int launch_status(const char* what) {
  cudaError_t e = cudaPeekAtLastError();
  if (e != cudaSuccess) {
    cudaGetLastError();
    return fail(ATMA_ERR_CUDA, "%s launch failed: %s", what, cudaGetErrorString(e));
  }
  return ATMA_OK;
}

// SM count of the calling thread's current device (148 when the query fails); read once per device.
inline int sm_count_of_current_device() {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) return 148;
    cached[dev] = n;                     // the same value from every host thread
  }
  return cached[dev];
}

inline size_t dtype_size(int dt) { return dt == ATMA_F32 ? 4 : 2; }
inline bool dtype_ok(int dt) { return dt == ATMA_F32 || dt == ATMA_BF16 || dt == ATMA_F16; }

// ---- device-side scalar conversions ------------------------------------------------
template <typename T> __device__ __forceinline__ float to_f32(T x);
template <> __device__ __forceinline__ float to_f32<float>(float x) { return x; }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 x) { return __bfloat162float(x); }
template <> __device__ __forceinline__ float to_f32<__half>(__half x) { return __half2float(x); }

template <typename T> __device__ __forceinline__ T from_f32(float x);
template <> __device__ __forceinline__ float from_f32<float>(float x) { return x; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float x) { return __float2bfloat16_rn(x); }
template <> __device__ __forceinline__ __half from_f32<__half>(float x) { return __float2half_rn(x); }

// Round an fp32 value through T and back (the rounding an eager op on a T tensor applies).
template <typename T> __device__ __forceinline__ float round_through(float x) { return to_f32<T>(from_f32<T>(x)); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Dispatch a lambda-like macro over the three supported element types.
#define ATMA_DISPATCH_DTYPE(dt, T, ...)                         \
  do {                                                          \
    if ((dt) == ATMA_F32) { using T = float; __VA_ARGS__; }     \
    else if ((dt) == ATMA_BF16) { using T = __nv_bfloat16; __VA_ARGS__; } \
    else { using T = __half; __VA_ARGS__; }                     \
  } while (0)

}  // namespace atma
