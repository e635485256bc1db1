// Warp-level tensor-core helpers (mma.sync m16n8k16, ldmatrix, cp.async) for the kernels whose
// working set is a small per-warp tile that must stay in registers across a recurrence:
// the gated-delta scan and the paged decode.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cstdint>

namespace atma {
namespace mma {

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// 16-byte chunk swizzle for a row-major 16-bit tile: chunk c of row r lives at chunk c ^ (r & 7),
// which makes the eight row addresses of one ldmatrix 8x8 matrix fall into distinct bank groups.
__device__ __forceinline__ int swz(int row, int chunk) { return chunk ^ (row & 7); }

// byte offset of element (row, col) in a swizzled tile whose rows hold `row_elems` 16-bit values
// (32, 64 or 128).  Rows of 64 bytes share a 128-byte line in pairs, so they swizzle on row/2.
__device__ __forceinline__ uint32_t tile_off(int row, int col, int row_elems) {
  const int sw = (row_elems >= 64) ? (row & 7) : ((row >> 1) & 3);
  return (uint32_t)(row * row_elems * 2 + (((col >> 3) ^ sw) << 4) + ((col & 7) << 1));
}

__device__ __forceinline__ void cp_async16(uint32_t smem_dst, const void* gsrc, bool valid) {
  const int n = valid ? 16 : 0;                      // 0 source bytes -> the 16 bytes are zero-filled
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_dst), "l"(gsrc), "r"(n) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t addr, uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}

// D (16x8 fp32) += A (16x16) * B (16x8); 16-bit operands, fp32 accumulate.
template <bool kBf16>
__device__ __forceinline__ void mma16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  if constexpr (kBf16) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  } else {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  }
}

template <bool kBf16>
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  if constexpr (kBf16) {
    __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
  } else {
    __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
  }
}
template <bool kBf16>
__device__ __forceinline__ float2 unpack2(uint32_t v) {
  if constexpr (kBf16) {
    return make_float2(__uint_as_float(v << 16), __uint_as_float(v & 0xffff0000u));
  } else {
    return __half22float2(*reinterpret_cast<__half2*>(&v));
  }
}

// ---- fragment address helpers (lane -> row / column of the 8x8 matrix it addresses) ------------
// A operand (16 x 16) from a row-major [m][k] tile: matrices (m0-7,k0-7) (m8-15,k0-7) (m0-7,k8-15) (m8-15,k8-15)
__device__ __forceinline__ void a_rowmajor_lane(int lane, int& m, int& k) { m = (lane & 7) + ((lane >> 3) & 1) * 8; k = (lane >> 4) * 8; }
// B operand, two n-tiles (16 n x 16 k), from a row-major [n][k] tile (k contiguous), no transpose:
// matrices (n0-7,k0-7) (n0-7,k8-15) (n8-15,k0-7) (n8-15,k8-15) -> r0,r1 = n-tile 0 (b0,b1); r2,r3 = n-tile 1
__device__ __forceinline__ void b_nk_lane(int lane, int& n, int& k) { n = (lane & 7) + (lane >> 4) * 8; k = ((lane >> 3) & 1) * 8; }
// B operand, two n-tiles, from a row-major [k][n] tile (n contiguous), with .trans:
// matrices (k0-7,n0-7) (k8-15,n0-7) (k0-7,n8-15) (k8-15,n8-15) -> r0,r1 = n-tile 0; r2,r3 = n-tile 1
__device__ __forceinline__ void b_kn_lane(int lane, int& k, int& n) { k = (lane & 7) + ((lane >> 3) & 1) * 8; n = (lane >> 4) * 8; }
// A operand (16 m x 16 k) from a tile stored [k][m] (m contiguous), with .trans:
// matrices a0 (k0-7,m0-7) a1 (k0-7,m8-15) a2 (k8-15,m0-7) a3 (k8-15,m8-15)
__device__ __forceinline__ void a_km_lane(int lane, int& k, int& m) { k = (lane & 7) + (lane >> 4) * 8; m = ((lane >> 3) & 1) * 8; }

}  // namespace mma
}  // namespace atma
