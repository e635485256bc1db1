// The two gate epilogues of a global layer's mixing output, each one pass instead of three eager ops
// (inference/models/atma.py:552-558 `_combine`: c * sigmoid(gate) before W_o; :246-252,373-375 the
// memory read-out: RMSNorm(r) * sigmoid(gate(x)) before mem.proj).  Both are bandwidth-bound
// elementwise kernels: 8 consecutive channels per thread (16-byte accesses for 16-bit types), every
// operand read once, the result written once.  Each value is rounded to the activation dtype where
// the separate eager ops would round (after the sigmoid, after the norm, after the product).
#include "common.cuh"

namespace atma {

namespace {

template <typename T> __device__ __forceinline__ void ep_load8(const T* p, float (&o)[8]) {
  if constexpr (sizeof(T) == 4) {
    const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
    o[0] = a.x; o[1] = a.y; o[2] = a.z; o[3] = a.w; o[4] = b.x; o[5] = b.y; o[6] = b.z; o[7] = b.w;
  } else {
    T v[8];
    *reinterpret_cast<uint4*>(v) = *reinterpret_cast<const uint4*>(p);
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j] = to_f32(v[j]);
  }
}

template <typename T> __device__ __forceinline__ void ep_store8(T* p, const float (&v)[8]) {
  if constexpr (sizeof(T) == 4) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
    *reinterpret_cast<float4*>(p + 4) = make_float4(v[4], v[5], v[6], v[7]);
  } else {
    T o[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j] = from_f32<T>(v[j]);
    *reinterpret_cast<uint4*>(p) = *reinterpret_cast<uint4*>(o);
  }
}

__device__ __forceinline__ float sigmoid_f32(float x) { return 1.0f / (1.0f + __expf(-x)); }

// out[r][h][c] = x[r][h][c] * sigmoid(gate[r][h][c]); x and gate with (row, head) strides, out dense
template <typename T>
__global__ void sigmoid_gate_mul_kernel(const T* __restrict__ x, int64_t x_row, int64_t x_head,
                                        const T* __restrict__ gate, int64_t g_row, int64_t g_head,
                                        T* __restrict__ out, int rows, int H, int dk) {
  const int per_head = dk / 8;
  const int64_t total = (int64_t)rows * H * per_head;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int c = (int)(i % per_head) * 8;
    const int64_t rh = i / per_head;
    const int h = (int)(rh % H);
    const int64_t r = rh / H;
    float xv[8], gv[8], o[8];
    ep_load8<T>(x + r * x_row + h * x_head + c, xv);
    ep_load8<T>(gate + r * g_row + h * g_head + c, gv);
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j] = xv[j] * round_through<T>(sigmoid_f32(gv[j]));
    ep_store8<T>(out + (r * H + h) * dk + c, o);
  }
}

// out[r][h*dk + c] = RMSNorm_dk(x[r][h][:])[c] * sigmoid(gate[r][h*dk + c]); 16 threads per head row
template <typename T>
__global__ void rms_sigmoid_gate_kernel(const T* __restrict__ x, const T* __restrict__ gate, int64_t g_row,
                                        T* __restrict__ out, int64_t n_head_rows, int H, int dk, float eps) {
  const int li = threadIdx.x & 15;
  const uint32_t half_mask = 0xffffu << (16 * ((threadIdx.x >> 4) & 1));
  const int64_t groups = ((int64_t)gridDim.x * blockDim.x) >> 4;
  const int c = li * 8;
  const bool on = c < dk;
  const float inv_dk = 1.0f / (float)dk;
  // every 16-thread group of a warp runs the same number of iterations (the shuffles name only the own half)
  for (int64_t hr = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 4; hr < n_head_rows; hr += groups) {
    const int64_t r = hr / H;
    const int h = (int)(hr - r * H);
    float xv[8], gv[8], o[8];
    if (on) {
      ep_load8<T>(x + hr * dk + c, xv);
      ep_load8<T>(gate + r * g_row + (int64_t)h * dk + c, gv);
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) { xv[j] = 0.f; gv[j] = 0.f; }
    }
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) ss = fmaf(xv[j], xv[j], ss);
#pragma unroll
    for (int o2 = 8; o2 > 0; o2 >>= 1) ss += __shfl_xor_sync(half_mask, ss, o2, 16);
    const float rs = rsqrtf(ss * inv_dk + eps);
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j] = round_through<T>(xv[j] * rs) * round_through<T>(sigmoid_f32(gv[j]));
    if (on) ep_store8<T>(out + hr * dk + c, o);
  }
}

int grid_for(int64_t threads_needed) {
  const int64_t want = (threads_needed + 255) / 256;
  return (int)(want < 148 * 16 ? (want > 0 ? want : 1) : 148 * 16);
}

}  // namespace
}  // namespace atma

using namespace atma;

extern "C" int atma_sigmoid_gate_mul(const void* x, int64_t x_row_stride, int64_t x_head_stride, const void* gate,
                                     int64_t gate_row_stride, int64_t gate_head_stride, void* out, int rows, int H,
                                     int dk, int dtype, void* stream) {
  ATMA_REQUIRE(dtype_ok(dtype), "sigmoid_gate_mul: unsupported dtype %d", dtype);
  ATMA_REQUIRE(rows >= 0 && H > 0 && dk > 0 && dk % 8 == 0, "sigmoid_gate_mul: head_dim %d must be a multiple of 8", dk);
  ATMA_REQUIRE(x_row_stride % 8 == 0 && x_head_stride % 8 == 0 && gate_row_stride % 8 == 0 && gate_head_stride % 8 == 0 &&
                   (uintptr_t)x % 16 == 0 && (uintptr_t)gate % 16 == 0 && (uintptr_t)out % 16 == 0,
               "sigmoid_gate_mul: rows must be 16-byte aligned (pointers and strides in multiples of 8 elements)");
  if (rows == 0) return ATMA_OK;
  const int blocks = grid_for((int64_t)rows * H * (dk / 8));
  ATMA_DISPATCH_DTYPE(dtype, T, {
    sigmoid_gate_mul_kernel<T><<<blocks, 256, 0, (cudaStream_t)stream>>>((const T*)x, x_row_stride, x_head_stride, (const T*)gate,
                                                                         gate_row_stride, gate_head_stride, (T*)out, rows, H, dk);
  });
  return launch_status("sigmoid_gate_mul");
}

extern "C" int atma_rms_sigmoid_gate(const void* x, const void* gate, int64_t gate_row_stride, void* out, int rows, int H,
                                     int dk, float eps, int dtype, void* stream) {
  ATMA_REQUIRE(dtype_ok(dtype), "rms_sigmoid_gate: unsupported dtype %d", dtype);
  ATMA_REQUIRE(rows >= 0 && H > 0 && dk > 0 && dk % 8 == 0 && dk <= 128,
               "rms_sigmoid_gate: head_dim %d must be a multiple of 8, at most 128", dk);
  ATMA_REQUIRE(gate_row_stride % 8 == 0 && (uintptr_t)x % 16 == 0 && (uintptr_t)gate % 16 == 0 && (uintptr_t)out % 16 == 0,
               "rms_sigmoid_gate: rows must be 16-byte aligned");
  if (rows == 0) return ATMA_OK;
  const int64_t n_head_rows = (int64_t)rows * H;
  const int blocks = grid_for(n_head_rows * 16);
  ATMA_DISPATCH_DTYPE(dtype, T, {
    rms_sigmoid_gate_kernel<T><<<blocks, 256, 0, (cudaStream_t)stream>>>((const T*)x, (const T*)gate, gate_row_stride, (T*)out,
                                                                         n_head_rows, H, dk, eps);
  });
  return launch_status("rms_sigmoid_gate");
}
