// Paged Polar decode, key-range ("split") kernel for 16-bit caches: the HBM-bound version.
//
// One CTA streams the K and V rows of one key range of one (sequence, KV head) through a
// cp.async ring of 64-key tiles (16-byte copies, one page-table lookup per tile when a tile
// cannot straddle pages, rows past the range zero-filled).  The arithmetic is laid out
// "keys as rows": each warp owns 16 keys of the tile and computes S^T = K_w Q^T with
// mma.sync m16n8k16 - the (up to 8) query heads of the GQA group are the 8 columns, Q^T sits in
// 16 registers for the whole kernel - then P^T goes back in as the B operand of
// O^T += V_w^T P^T after an 8x8 register transpose (movmatrix).  Compared with heads-as-rows
// (16 rows, of which a GQA group fills 4) this halves the MMAs, the exponentials and the
// accumulator registers.  The running maximum of a head is only raised when some score exceeds
// it by more than 2^8 (one warp vote per tile), so the usual per-tile max reduction and
// rescale disappear from the steady state; L, Q2 and O stay relative to that reference.
// The four warps are merged once at the end and the partial statistics go to the scratch
// layout the merge kernel reads.
#include "common.cuh"
#include "mma_sync.cuh"

namespace atma {

using namespace mma;

namespace {

constexpr int kTileKeys = 64;
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;
constexpr float kNegBig = -1e38f;
constexpr float kRaise = 8.0f;                // log2 slack before the reference maximum is raised

__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t a) {
  uint32_t d;
  asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(d) : "r"(a));
  return d;
}

template <bool kBf16, int DK, int STAGES>
__global__ void __launch_bounds__(128, STAGES == 2 ? 3 : 2)
polar_decode_split_mma_kernel(const uint16_t* __restrict__ q, const uint16_t* __restrict__ k_cache,
                              const uint16_t* __restrict__ v_cache, const int32_t* __restrict__ block_tables,
                              int64_t bt_stride, const int32_t* __restrict__ context_lens, const int32_t* __restrict__ temp_lens,
                              const float* __restrict__ spg, float* __restrict__ scratch, int B, int H, int Hkv,
                              int block_size, int max_blocks, int num_blocks, int n_splits, int window,
                              const uint16_t* __restrict__ append_k, int64_t append_k_st, const uint16_t* __restrict__ append_v,
                              int64_t append_v_st, const int32_t* __restrict__ append_slots) {
  constexpr int KS = DK / 16;                 // k-steps of K Q^T
  constexpr int MT = DK / 16;                 // m-tiles of V^T P^T
  constexpr int CH = DK / 8;                  // 16-byte chunks per row
  constexpr int kTileBytes = kTileKeys * DK * 2;
  constexpr int OLD = DK + 4;                 // row stride of the merge buffer (floats)
  extern __shared__ __align__(128) uint8_t sm[];
  uint8_t* KV = sm;                           // [STAGES][K tile | V tile]

  const int G = H / Hkv;
  const int ngrp = (G + 7) / 8;               // more than 8 heads per KV head: several CTAs share the rows
  const int split = blockIdx.x, kvh = blockIdx.y / ngrp, g0 = (blockIdx.y % ngrp) * 8, b = blockIdx.z;
  const int Gl = min(8, G - g0);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int gq = lane >> 2, tq = lane & 3;

  int n = context_lens[b];
  n = max(0, min(n, max_blocks * block_size));
  const int lo_w = window > 0 ? max(n - window, 0) : 0;
  int chunk = (n - lo_w + n_splits - 1) / n_splits;
  chunk = (chunk + kTileKeys - 1) / kTileKeys * kTileKeys;
  const int lo = lo_w + split * chunk;
  const int hi = min(lo + chunk, n);

  // The token being decoded: the CTA whose key range ends with it stores its K and V rows before anything of
  // the cache is read (16 bytes per thread; the fence and the barrier order the stores before this CTA's loads;
  // no other CTA of the launch reads that row, because the key ranges are disjoint).
  if (append_slots != nullptr) {
    if (hi == n && lo < hi && g0 == 0 && tid < 2 * CH) {
      const int cs = append_slots[b];
      if (cs >= 0) {
        const int isv = tid / CH, ch = tid % CH;
        const uint16_t* src = (isv ? append_v + b * append_v_st : append_k + b * append_k_st) + kvh * DK + ch * 8;
        uint16_t* dst = const_cast<uint16_t*>(isv ? v_cache : k_cache) + ((int64_t)cs * Hkv + kvh) * DK + ch * 8;
        *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(src);
        __threadfence();
      }
    }
    __syncthreads();
  }
  float* stats = scratch;
  float* sacc = scratch + (int64_t)B * H * n_splits * 4;
  if (lo >= hi) {                             // empty range: neutral partial
    for (int g = warp; g < Gl; g += 4) {
      const int64_t bh = (int64_t)b * H + kvh * G + g0 + g;
      if (lane == 0) *reinterpret_cast<float4*>(stats + (bh * n_splits + split) * 4) = make_float4(kNegBig, 0.f, 0.f, 0.f);
      for (int d = lane; d < DK; d += 32) sacc[(bh * n_splits + split) * DK + d] = 0.f;
    }
    return;
  }

  const int64_t row_stride = (int64_t)Hkv * DK;
  const int32_t* bt = block_tables + b * bt_stride;
  const int n_tiles = (hi - lo + kTileKeys - 1) / kTileKeys;
  const bool tile_in_page = (block_size % kTileKeys == 0) && (lo % kTileKeys == 0);

  auto load_tile = [&](int it) {
    uint8_t* dst = KV + (it % STAGES) * 2 * kTileBytes;
    const int pos0 = lo + it * kTileKeys;
    if (tile_in_page) {
      const int blk = pos0 / block_size;
      const int phys = min(max(bt[blk], 0), num_blocks - 1);
      const int64_t base = ((int64_t)phys * block_size + (pos0 - blk * block_size)) * row_stride + (int64_t)kvh * DK;
#pragma unroll
      for (int j = 0; j < kTileKeys * CH / 128; ++j) {
        const int i = tid + j * 128;
        const int r = i / CH, ch = i % CH;
        const bool ok = pos0 + r < hi;
        const int64_t off = ok ? base + r * row_stride + ch * 8 : 0;
        cp_async16(smem_u32(dst) + tile_off(r, ch * 8, DK), k_cache + off, ok);
        cp_async16(smem_u32(dst) + kTileBytes + tile_off(r, ch * 8, DK), v_cache + off, ok);
      }
    } else {
#pragma unroll
      for (int j = 0; j < kTileKeys * CH / 128; ++j) {
        const int i = tid + j * 128;
        const int r = i / CH, ch = i % CH;
        const int pos = pos0 + r;
        const bool ok = pos < hi;
        int64_t off = 0;
        if (ok) {
          const int blk = pos / block_size;
          const int phys = min(max(bt[blk], 0), num_blocks - 1);
          off = ((int64_t)phys * block_size + (pos - blk * block_size)) * row_stride + (int64_t)kvh * DK + ch * 8;
        }
        cp_async16(smem_u32(dst) + tile_off(r, ch * 8, DK), k_cache + off, ok);
        cp_async16(smem_u32(dst) + kTileBytes + tile_off(r, ch * 8, DK), v_cache + off, ok);
      }
    }
  };

#pragma unroll
  for (int s = 0; s < STAGES - 1; ++s) {
    if (s < n_tiles) load_tile(s);
    cp_async_commit();
  }

  // ---- Q^T as the B operand: column gq = head g0 + gq (zero beyond the group), rows = dims ------------
  uint32_t qb[KS][2];
  {
    const uint16_t* qrow = q + ((int64_t)b * H + kvh * G + g0 + (gq < Gl ? gq : 0)) * DK;
#pragma unroll
    for (int ks = 0; ks < KS; ++ks) {
      qb[ks][0] = (gq < Gl) ? *reinterpret_cast<const uint32_t*>(qrow + 16 * ks + 2 * tq) : 0u;
      qb[ks][1] = (gq < Gl) ? *reinterpret_cast<const uint32_t*>(qrow + 16 * ks + 8 + 2 * tq) : 0u;
    }
  }
  // this thread's two heads: g0 + 2 tq + e
  const int nt = temp_lens != nullptr ? temp_lens[b] : n;      // the whole context sets the temperature
  const float nf = fmaxf(window > 0 ? fminf((float)nt, (float)window) : (float)nt, 1.0f);
  const float logn = logf(nf);
  float sc[2];                                 // log2-domain score scale
#pragma unroll
  for (int e = 0; e < 2; ++e) {
    const int g = 2 * tq + e;
    sc[e] = (g < Gl) ? (1.0f + spg[kvh * G + g0 + g] * logn) * rsqrtf((float)DK) * kLog2e : 0.f;
  }

  float mref[2] = {kNegBig, kNegBig}, L[2] = {0.f, 0.f}, Q2[2] = {0.f, 0.f};   // L, Q2: this thread's keys only
  float O[MT][4];                              // O^T: [dim gq | gq + 8 of m-tile][head 2tq + e]
#pragma unroll
  for (int mt = 0; mt < MT; ++mt)
#pragma unroll
    for (int e = 0; e < 4; ++e) O[mt][e] = 0.f;
  int am, ak, vk, vm;
  a_rowmajor_lane(lane, am, ak);
  a_km_lane(lane, vk, vm);

  for (int it = 0; it < n_tiles; ++it) {
    cp_async_wait<STAGES - 2>();
    __syncthreads();                           // tile `it` landed; everyone is done with tile it-1
    if (it + STAGES - 1 < n_tiles) load_tile(it + STAGES - 1);
    cp_async_commit();
    const uint32_t Ksm = smem_u32(KV + (it % STAGES) * 2 * kTileBytes), Vsm = Ksm + kTileBytes;

    // S^T (16 keys of this warp x 8 heads)
    float S[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int ks = 0; ks < KS; ++ks) {
      uint32_t af[4];
      ldsm_x4(Ksm + tile_off(16 * warp + am, 16 * ks + ak, DK), af);
      mma16816<kBf16>(S, af, qb[ks][0], qb[ks][1]);
    }
    const int key0 = lo + it * kTileKeys + 16 * warp + gq;
    const bool ok0 = key0 < hi, ok1 = key0 + 8 < hi;
    float a[4];                                // [key gq][e], [key gq + 8][e]
    a[0] = ok0 ? S[0] * sc[0] : -INFINITY; a[1] = ok0 ? S[1] * sc[1] : -INFINITY;
    a[2] = ok1 ? S[2] * sc[0] : -INFINITY; a[3] = ok1 ? S[3] * sc[1] : -INFINITY;
    float mx[2] = {fmaxf(a[0], a[2]), fmaxf(a[1], a[3])};
    if (__any_sync(0xffffffffu, mx[0] > mref[0] + kRaise || mx[1] > mref[1] + kRaise)) {
#pragma unroll
      for (int e = 0; e < 2; ++e) {            // raise the reference maximum of the heads (whole warp)
        float w = mx[e];
        w = fmaxf(w, __shfl_xor_sync(0xffffffffu, w, 4));
        w = fmaxf(w, __shfl_xor_sync(0xffffffffu, w, 8));
        w = fmaxf(w, __shfl_xor_sync(0xffffffffu, w, 16));
        const float m_new = fmaxf(mref[e], w);
        const float alpha = exp2f(mref[e] - m_new);
        L[e] *= alpha; Q2[e] *= alpha * alpha;
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) { O[mt][e] *= alpha; O[mt][2 + e] *= alpha; }
        mref[e] = m_new;
      }
    }
    float p[4];
    p[0] = exp2f(a[0] - mref[0]); p[1] = exp2f(a[1] - mref[1]);
    p[2] = exp2f(a[2] - mref[0]); p[3] = exp2f(a[3] - mref[1]);
    L[0] += p[0] + p[2]; L[1] += p[1] + p[3];
    Q2[0] = fmaf(p[0], p[0], fmaf(p[2], p[2], Q2[0]));
    Q2[1] = fmaf(p[1], p[1], fmaf(p[3], p[3], Q2[1]));
    // P^T as the B operand: rows = keys, columns = heads
    const uint32_t pb0 = movmatrix_trans(pack2<kBf16>(p[0], p[1]));
    const uint32_t pb1 = movmatrix_trans(pack2<kBf16>(p[2], p[3]));
    // O^T += V_w^T P^T
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
      uint32_t af[4];
      ldsm_x4_trans(Vsm + tile_off(16 * warp + vk, 16 * mt + vm, DK), af);
      mma16816<kBf16>(O[mt], af, pb0, pb1);
    }
  }
  cp_async_wait<0>();
  __syncthreads();                             // the stage buffers are free: reuse them for the merge

  // ---- merge the four warps ------------------------------------------------------------------------
  float* s_o = reinterpret_cast<float*>(KV);                   // [4 warps][8 heads][OLD]
  float* s_m = s_o + 4 * 8 * OLD;                              // [4][8]
  float* s_l = s_m + 32;
  float* s_q2 = s_l + 32;
#pragma unroll
  for (int e = 0; e < 2; ++e) {
    L[e] += __shfl_xor_sync(0xffffffffu, L[e], 4); L[e] += __shfl_xor_sync(0xffffffffu, L[e], 8);
    L[e] += __shfl_xor_sync(0xffffffffu, L[e], 16);
    Q2[e] += __shfl_xor_sync(0xffffffffu, Q2[e], 4); Q2[e] += __shfl_xor_sync(0xffffffffu, Q2[e], 8);
    Q2[e] += __shfl_xor_sync(0xffffffffu, Q2[e], 16);
    if (gq == 0) s_m[warp * 8 + 2 * tq + e] = mref[e];
  }
  __syncthreads();
#pragma unroll
  for (int e = 0; e < 2; ++e) {
    const int g = 2 * tq + e;
    const float M = fmaxf(fmaxf(s_m[g], s_m[8 + g]), fmaxf(s_m[16 + g], s_m[24 + g]));
    const float w = exp2f(mref[e] - M);
    if (gq == 0) { s_l[warp * 8 + g] = L[e] * w; s_q2[warp * 8 + g] = Q2[e] * w * w; }
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
      s_o[(warp * 8 + g) * OLD + 16 * mt + gq] = O[mt][e] * w;
      s_o[(warp * 8 + g) * OLD + 16 * mt + gq + 8] = O[mt][2 + e] * w;
    }
  }
  __syncthreads();
  for (int i = tid; i < Gl * DK; i += 128) {
    const int g = i / DK, d = i - g * DK;
    const float s = s_o[g * OLD + d] + s_o[(8 + g) * OLD + d] + s_o[(16 + g) * OLD + d] + s_o[(24 + g) * OLD + d];
    const int64_t bh = (int64_t)b * H + kvh * G + g0 + g;
    sacc[(bh * n_splits + split) * DK + d] = s;
  }
  if (tid < Gl) {
    const int g = tid;
    const float M = fmaxf(fmaxf(s_m[g], s_m[8 + g]), fmaxf(s_m[16 + g], s_m[24 + g]));
    const float l = s_l[g] + s_l[8 + g] + s_l[16 + g] + s_l[24 + g];
    const float q2 = s_q2[g] + s_q2[8 + g] + s_q2[16 + g] + s_q2[24 + g];
    const int64_t bh = (int64_t)b * H + kvh * G + g0 + g;
    // the merge kernel works with natural-log maxima
    *reinterpret_cast<float4*>(stats + (bh * n_splits + split) * 4) = make_float4(M <= -1e37f ? kNegBig : M * kLn2, l, q2, 0.f);
  }
}

}  // namespace

bool polar_decode_mma_supported(const atma_polar_decode_args& a) {
  const int G = a.H / a.Hkv;
  return (a.dtype == ATMA_BF16 || a.dtype == ATMA_F16) && (a.dk == 128 || a.dk == 64) && G <= 16;
}

// Whether the key-range kernel stores the token's own K/V rows (one CTA group per KV head, so that no other CTA
// reads the row that is being written).
bool polar_decode_mma_appends(const atma_polar_decode_args& a) {
  return polar_decode_mma_supported(a) && a.append_k != nullptr && a.append_v != nullptr && a.append_slots != nullptr &&
         a.H / a.Hkv <= 8 && (reinterpret_cast<uintptr_t>(a.append_k) & 15) == 0 && (reinterpret_cast<uintptr_t>(a.append_v) & 15) == 0 &&
         a.append_k_stride % 8 == 0 && a.append_v_stride % 8 == 0;
}

int polar_decode_split_mma(const atma_polar_decode_args& a, cudaStream_t st) {
  const int G = a.H / a.Hkv;
  dim3 grid(a.n_splits, a.Hkv * ((G + 7) / 8), a.B);
  constexpr int kStages = 3;                  // 3 x 32 KB per CTA, two CTAs per SM: ~200 KB of loads in flight per SM
  const int smem = kStages * 2 * kTileKeys * a.dk * 2;
  const void* ak = polar_decode_mma_appends(a) ? a.append_k : nullptr;
#define ATMA_LAUNCH(BF, DKK)                                                                                    \
  do {                                                                                                          \
    auto kern = polar_decode_split_mma_kernel<BF, DKK, kStages>;                                                \
    ATMA_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));                \
    kern<<<grid, 128, smem, st>>>((const uint16_t*)a.q, (const uint16_t*)a.k_cache, (const uint16_t*)a.v_cache, \
                                  a.block_tables, a.bt_stride, a.context_lens, a.temp_lens, a.spg, a.scratch, a.B, a.H,      \
                                  a.Hkv, a.block_size, a.max_blocks, a.num_blocks, a.n_splits, a.window,        \
                                  (const uint16_t*)ak, a.append_k_stride, (const uint16_t*)a.append_v, a.append_v_stride, \
                                  ak ? a.append_slots : nullptr);                                               \
  } while (0)
  if (a.dtype == ATMA_BF16) { if (a.dk == 128) ATMA_LAUNCH(true, 128); else ATMA_LAUNCH(true, 64); }
  else { if (a.dk == 128) ATMA_LAUNCH(false, 128); else ATMA_LAUNCH(false, 64); }
#undef ATMA_LAUNCH
  return launch_status("polar_decode (split, mma)");
}

}  // namespace atma
