// Bandwidth-bound elementwise kernels of the decode path: squared-ReLU gate, logit
// soft-cap, KV-cache scatter.  Also hosts the library's error-message plumbing.
#include "common.cuh"

namespace atma {

char* err_buf() {
  static thread_local char buf[512] = {0};
  return buf;
}

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(err_buf(), 512, fmt, ap);
  va_end(ap);
  return code;
}

// ---- gate * relu(x)^2 ------------------------------------------------------------------
// One thread handles VEC consecutive columns of one row (16-byte loads when aligned).
template <typename T, int VEC>
__global__ void squared_relu_gate_kernel(const T* __restrict__ x, int64_t x_stride,
                                         const T* __restrict__ gate, int64_t gate_stride,
                                         T* __restrict__ out, int rows, int width) {
  const int vec_per_row = width / VEC;
  const int64_t total = (int64_t)rows * vec_per_row;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (int64_t)gridDim.x * blockDim.x) {
    const int row = (int)(i / vec_per_row);
    const int col = (int)(i - (int64_t)row * vec_per_row) * VEC;
    T xv[VEC], gv[VEC], ov[VEC];
    if constexpr (VEC * sizeof(T) == 16) {
      *reinterpret_cast<uint4*>(xv) = *reinterpret_cast<const uint4*>(x + row * x_stride + col);
      *reinterpret_cast<uint4*>(gv) = *reinterpret_cast<const uint4*>(gate + row * gate_stride + col);
    } else {
#pragma unroll
      for (int j = 0; j < VEC; ++j) { xv[j] = x[row * x_stride + col + j]; gv[j] = gate[row * gate_stride + col + j]; }
    }
#pragma unroll
    for (int j = 0; j < VEC; ++j) {
      float p = fmaxf(to_f32(xv[j]), 0.f);
      float sq = p * p;
      // Eager bf16 materialises relu(x)^2 as a bf16 tensor before the gate multiply.
      if constexpr (sizeof(T) == 2 && !std::is_same<T, __half>::value) sq = round_through<T>(sq);
      ov[j] = from_f32<T>(to_f32(gv[j]) * sq);
    }
    if constexpr (VEC * sizeof(T) == 16) {
      *reinterpret_cast<uint4*>(out + (int64_t)row * width + col) = *reinterpret_cast<uint4*>(ov);
    } else {
#pragma unroll
      for (int j = 0; j < VEC; ++j) out[(int64_t)row * width + col + j] = ov[j];
    }
  }
}

// ---- 15 x / sqrt(x^2 + 225) ------------------------------------------------------------
template <typename T>
__global__ void softcap_kernel(const T* __restrict__ x, T* __restrict__ out, int64_t n) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (int64_t)gridDim.x * blockDim.x) {
    float v = to_f32(x[i]);
    float left = 15.0f * v, sq = v * v;
    constexpr bool kRound = std::is_same<T, __nv_bfloat16>::value;
    if constexpr (kRound) { left = round_through<T>(left); sq = round_through<T>(sq); }
    float den = sq + 225.0f;
    if constexpr (kRound) den = round_through<T>(den);
    float inv = rsqrtf(den);
    if constexpr (kRound) inv = round_through<T>(inv);
    out[i] = from_f32<T>(left * inv);
  }
}

// ---- paged KV-cache scatter: one CTA per new token, 16-byte copies ------------------------
__global__ void store_kvcache_kernel(const char* __restrict__ key, int64_t key_stride_b,
                                     const char* __restrict__ value, int64_t value_stride_b,
                                     char* __restrict__ k_cache, char* __restrict__ v_cache,
                                     const int32_t* __restrict__ slot_mapping, int row_bytes) {
  const int i = blockIdx.x;
  const int slot = slot_mapping[i];
  if (slot < 0) return;
  const char* ks = key + i * key_stride_b;
  const char* vs = value + i * value_stride_b;
  char* kd = k_cache + (int64_t)slot * row_bytes;
  char* vd = v_cache + (int64_t)slot * row_bytes;
  for (int o = threadIdx.x * 16; o < row_bytes; o += blockDim.x * 16) {
    *reinterpret_cast<uint4*>(kd + o) = *reinterpret_cast<const uint4*>(ks + o);
    *reinterpret_cast<uint4*>(vd + o) = *reinterpret_cast<const uint4*>(vs + o);
  }
}

__global__ void store_kvcache_kernel_bytes2(const char* __restrict__ key, int64_t key_stride_b,
                                            const char* __restrict__ value, int64_t value_stride_b,
                                            char* __restrict__ k_cache, char* __restrict__ v_cache,
                                            const int32_t* __restrict__ slot_mapping, int row_bytes) {
  const int i = blockIdx.x;
  const int slot = slot_mapping[i];
  if (slot < 0) return;
  for (int o = threadIdx.x * 2; o < row_bytes; o += blockDim.x * 2) {
    *reinterpret_cast<uint16_t*>(k_cache + (int64_t)slot * row_bytes + o) =
        *reinterpret_cast<const uint16_t*>(key + i * key_stride_b + o);
    *reinterpret_cast<uint16_t*>(v_cache + (int64_t)slot * row_bytes + o) =
        *reinterpret_cast<const uint16_t*>(value + i * value_stride_b + o);
  }
}

}  // namespace atma

using namespace atma;

extern "C" const char* atma_last_error(void) { return err_buf(); }
extern "C" int atma_abi_version(void) { return 1; }

extern "C" int atma_squared_relu_gate(const void* x, int64_t x_stride, const void* gate,
                                      int64_t gate_stride, void* out, int rows, int width,
                                      int dtype, void* stream) {
  ATMA_REQUIRE(dtype_ok(dtype), "squared_relu_gate: unsupported dtype %d", dtype);
  ATMA_REQUIRE(rows >= 0 && width >= 0, "squared_relu_gate: negative shape");
  if (rows == 0 || width == 0) return ATMA_OK;
  cudaStream_t st = (cudaStream_t)stream;
  const size_t es = dtype_size(dtype);
  const int vec = (int)(16 / es);
  const bool aligned = (width % vec == 0) && (x_stride % vec == 0) && (gate_stride % vec == 0) &&
                       ((uintptr_t)x % 16 == 0) && ((uintptr_t)gate % 16 == 0) && ((uintptr_t)out % 16 == 0);
  const int64_t work = (int64_t)rows * (aligned ? width / vec : width);
  const int threads = 256;
  const int blocks = (int)((work + threads - 1) / threads < 148 * 16 ? (work + threads - 1) / threads : 148 * 16);
  ATMA_DISPATCH_DTYPE(dtype, T, {
    if (aligned)
      squared_relu_gate_kernel<T, 16 / sizeof(T)><<<blocks, threads, 0, st>>>(
          (const T*)x, x_stride, (const T*)gate, gate_stride, (T*)out, rows, width);
    else
      squared_relu_gate_kernel<T, 1><<<blocks, threads, 0, st>>>(
          (const T*)x, x_stride, (const T*)gate, gate_stride, (T*)out, rows, width);
  });
  return launch_status("squared_relu_gate");
}

extern "C" int atma_softcap_logits(const void* x, void* out, int64_t n, int dtype, void* stream) {
  ATMA_REQUIRE(dtype_ok(dtype), "softcap_logits: unsupported dtype %d", dtype);
  if (n <= 0) return ATMA_OK;
  const int threads = 256;
  int64_t want = (n + threads - 1) / threads;
  const int blocks = (int)(want < 148 * 16 ? want : 148 * 16);
  ATMA_DISPATCH_DTYPE(dtype, T, {
    softcap_kernel<T><<<blocks, threads, 0, (cudaStream_t)stream>>>((const T*)x, (T*)out, n);
  });
  return launch_status("softcap_logits");
}

extern "C" int atma_store_kvcache(const void* key, int64_t key_stride, const void* value,
                                  int64_t value_stride, void* k_cache, void* v_cache,
                                  const int32_t* slot_mapping, int N, int D, int elem_size,
                                  void* stream) {
  ATMA_REQUIRE(elem_size == 2 || elem_size == 4, "store_kvcache: element size %d", elem_size);
  if (N <= 0 || D <= 0) return ATMA_OK;
  const int row_bytes = D * elem_size;
  const bool vec = (row_bytes % 16 == 0) && ((key_stride * elem_size) % 16 == 0) &&
                   ((value_stride * elem_size) % 16 == 0) && ((uintptr_t)key % 16 == 0) &&
                   ((uintptr_t)value % 16 == 0) && ((uintptr_t)k_cache % 16 == 0) &&
                   ((uintptr_t)v_cache % 16 == 0);
  if (vec)
    store_kvcache_kernel<<<N, 64, 0, (cudaStream_t)stream>>>(
        (const char*)key, key_stride * elem_size, (const char*)value, value_stride * elem_size,
        (char*)k_cache, (char*)v_cache, slot_mapping, row_bytes);
  else
    store_kvcache_kernel_bytes2<<<N, 64, 0, (cudaStream_t)stream>>>(
        (const char*)key, key_stride * elem_size, (const char*)value, value_stride * elem_size,
        (char*)k_cache, (char*)v_cache, slot_mapping, row_bytes);
  return launch_status("store_kvcache");
}
