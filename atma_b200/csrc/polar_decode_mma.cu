// Paged Polar decode, key-range ("split") kernel for 16-bit caches: the HBM-bound version.
//
// One CTA streams the K and V rows of one key range of one (sequence, KV head) through a
// 3-stage cp.async ring of 64-key tiles (page-table lookup per row, 16-byte copies, rows past
// the range zero-filled), so that two CTAs per SM keep >100 KB of loads in flight.  The G query
// heads of the GQA group are the rows of a 16-row tile: each warp multiplies it with its 16
// keys of the tile on the tensor cores (mma.sync m16n8k16), keeps running (m, L, Q2, O) for
// those keys in registers, and feeds P straight from the accumulator registers into the P V
// product.  With the arithmetic on the tensor pipe the CUDA cores only do the exponentials,
// and the kernel is limited by the cache read.  The four warps are merged once at the end and
// the partial statistics go to the same scratch layout the merge kernel reads.
#include "common.cuh"
#include "mma_sync.cuh"

namespace atma {

using namespace mma;

namespace {

constexpr int kTileKeys = 64;
constexpr int kStages = 3;
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;
constexpr float kNegBig = -1e38f;

template <bool kBf16, int DK>
__global__ void __launch_bounds__(128, 2)
polar_decode_split_mma_kernel(const uint16_t* __restrict__ q, const uint16_t* __restrict__ k_cache,
                              const uint16_t* __restrict__ v_cache, const int32_t* __restrict__ block_tables,
                              int64_t bt_stride, const int32_t* __restrict__ context_lens,
                              const float* __restrict__ spg, float* __restrict__ scratch, int B, int H, int Hkv,
                              int block_size, int max_blocks, int num_blocks, int n_splits, int window) {
  constexpr int KS = DK / 16;                 // k-steps of Q K^T
  constexpr int NT = DK / 8;                  // n-tiles of P V
  constexpr int CH = DK / 8;                  // 16-byte chunks per row
  constexpr int kTileBytes = kTileKeys * DK * 2;
  extern __shared__ __align__(128) uint8_t sm[];
  uint8_t* Qs = sm;                           // [16][DK]
  uint8_t* KV = sm + 16 * DK * 2;             // [kStages][K tile | V tile]

  const int split = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
  const int G = H / Hkv;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int gq = lane >> 2, tq = lane & 3;

  int n = context_lens[b];
  n = max(0, min(n, max_blocks * block_size));
  const int lo_w = window > 0 ? max(n - window, 0) : 0;
  int chunk = (n - lo_w + n_splits - 1) / n_splits;
  chunk = (chunk + kTileKeys - 1) / kTileKeys * kTileKeys;
  const int lo = lo_w + split * chunk;
  const int hi = min(lo + chunk, n);

  float* stats = scratch;
  float* sacc = scratch + (int64_t)B * H * n_splits * 4;
  if (lo >= hi) {                             // empty range: neutral partial
    for (int g = warp; g < G; g += 4) {
      const int64_t bh = (int64_t)b * H + kvh * G + g;
      if (lane == 0) *reinterpret_cast<float4*>(stats + (bh * n_splits + split) * 4) = make_float4(kNegBig, 0.f, 0.f, 0.f);
      for (int d = lane; d < DK; d += 32) sacc[(bh * n_splits + split) * DK + d] = 0.f;
    }
    return;
  }

  // ---- Q rows (zero beyond the G real heads) -----------------------------------------------------
  for (int i = tid; i < 16 * CH; i += 128) {
    const int r = i / CH, ch = i % CH;
    uint4 val = make_uint4(0u, 0u, 0u, 0u);
    if (r < G) val = *reinterpret_cast<const uint4*>(q + ((int64_t)b * H + kvh * G + r) * DK + ch * 8);
    *reinterpret_cast<uint4*>(Qs + tile_off(r, ch * 8, DK)) = val;
  }
  const float nf = fmaxf(window > 0 ? fminf((float)n, (float)window) : (float)n, 1.0f);
  const float logn = logf(nf);
  float sc[2];                                 // log2-domain score scale of rows gq and gq + 8
#pragma unroll
  for (int hh = 0; hh < 2; ++hh) {
    const int r = gq + 8 * hh;
    sc[hh] = (r < G) ? (1.0f + spg[kvh * G + r] * logn) * rsqrtf((float)DK) * kLog2e : 0.f;
  }

  const int64_t row_stride = (int64_t)Hkv * DK;
  const int32_t* bt = block_tables + b * bt_stride;
  const int n_tiles = (hi - lo + kTileKeys - 1) / kTileKeys;

  auto load_tile = [&](int it) {
    uint8_t* dst = KV + (it % kStages) * 2 * kTileBytes;
    const int pos0 = lo + it * kTileKeys;
#pragma unroll
    for (int j = 0; j < kTileKeys * CH / 128; ++j) {
      const int i = tid + j * 128;
      const int r = i / CH, ch = i % CH;
      const int pos = pos0 + r;
      const bool ok = pos < hi;
      int64_t off = 0;
      if (ok) {
        const int blk = pos / block_size;
        int phys = bt[blk];
        phys = min(max(phys, 0), num_blocks - 1);
        off = ((int64_t)phys * block_size + (pos - blk * block_size)) * row_stride + (int64_t)kvh * DK + ch * 8;
      }
      cp_async16(smem_u32(dst) + tile_off(r, ch * 8, DK), k_cache + off, ok);
      cp_async16(smem_u32(dst) + kTileBytes + tile_off(r, ch * 8, DK), v_cache + off, ok);
    }
  };

#pragma unroll
  for (int s = 0; s < kStages - 1; ++s) {
    if (s < n_tiles) load_tile(s);
    cp_async_commit();
  }
  __syncthreads();                             // Qs visible
  uint32_t qa[KS][4];
  {
    int am, ak;
    a_rowmajor_lane(lane, am, ak);
#pragma unroll
    for (int ks = 0; ks < KS; ++ks) ldsm_x4(smem_u32(Qs) + tile_off(am, 16 * ks + ak, DK), qa[ks]);
  }

  float m[2] = {kNegBig, kNegBig}, L[2] = {0.f, 0.f}, Q2[2] = {0.f, 0.f};
  float O[NT][4];
#pragma unroll
  for (int nt = 0; nt < NT; ++nt)
#pragma unroll
    for (int e = 0; e < 4; ++e) O[nt][e] = 0.f;
  int bn, bk, vk, vn;
  b_nk_lane(lane, bn, bk);
  b_kn_lane(lane, vk, vn);

  for (int it = 0; it < n_tiles; ++it) {
    cp_async_wait<kStages - 2>();
    __syncthreads();                           // tile `it` landed; everyone is done with tile it-1
    if (it + kStages - 1 < n_tiles) load_tile(it + kStages - 1);
    cp_async_commit();
    const uint32_t Ksm = smem_u32(KV + (it % kStages) * 2 * kTileBytes), Vsm = Ksm + kTileBytes;

    // S (16 heads x 16 keys of this warp)
    float S[2][4];
#pragma unroll
    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) S[nt][e] = 0.f;
#pragma unroll
    for (int ks = 0; ks < KS; ++ks) {
      uint32_t bf[4];
      ldsm_x4(Ksm + tile_off(16 * warp + bn, 16 * ks + bk, DK), bf);
      mma16816<kBf16>(S[0], qa[ks], bf[0], bf[1]);
      mma16816<kBf16>(S[1], qa[ks], bf[2], bf[3]);
    }
    // online softmax statistics for rows gq (hh = 0) and gq + 8 (hh = 1)
    const int key0 = lo + it * kTileKeys + 16 * warp;
    uint32_t pa[4];
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
      float a[4];
#pragma unroll
      for (int nt = 0; nt < 2; ++nt)
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int pos = key0 + 8 * nt + 2 * tq + e;
          a[2 * nt + e] = (pos < hi) ? S[nt][2 * hh + e] * sc[hh] : -INFINITY;
        }
      float mx = fmaxf(fmaxf(a[0], a[1]), fmaxf(a[2], a[3]));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
      const float m_new = fmaxf(m[hh], mx);
      const float alpha = exp2f(m[hh] - m_new);
      float p[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) p[e] = exp2f(a[e] - m_new);
      L[hh] = L[hh] * alpha + (p[0] + p[1]) + (p[2] + p[3]);
      Q2[hh] = Q2[hh] * alpha * alpha + fmaf(p[0], p[0], p[1] * p[1]) + fmaf(p[2], p[2], p[3] * p[3]);
      m[hh] = m_new;
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) { O[nt][2 * hh] *= alpha; O[nt][2 * hh + 1] *= alpha; }
      pa[hh] = pack2<kBf16>(p[0], p[1]);       // a0 / a1: keys 2t,2t+1 of n-tile 0
      pa[2 + hh] = pack2<kBf16>(p[2], p[3]);   // a2 / a3: keys 8+2t.. (n-tile 1)
    }
    // O += P V  (16 keys of this warp)
#pragma unroll
    for (int pr = 0; pr < NT / 2; ++pr) {
      uint32_t bf[4];
      ldsm_x4_trans(Vsm + tile_off(16 * warp + vk, 16 * pr + vn, DK), bf);
      mma16816<kBf16>(O[2 * pr], pa, bf[0], bf[1]);
      mma16816<kBf16>(O[2 * pr + 1], pa, bf[2], bf[3]);
    }
  }
  cp_async_wait<0>();
  __syncthreads();                             // the stage buffers are free: reuse them for the merge

  // ---- merge the four warps ------------------------------------------------------------------------
  float* s_o = reinterpret_cast<float*>(KV);                   // [4][16][DK]
  float* s_m = s_o + 4 * 16 * DK;                              // [4][16]
  float* s_l = s_m + 64;
  float* s_q2 = s_l + 64;
#pragma unroll
  for (int hh = 0; hh < 2; ++hh) {
    L[hh] += __shfl_xor_sync(0xffffffffu, L[hh], 1); L[hh] += __shfl_xor_sync(0xffffffffu, L[hh], 2);
    Q2[hh] += __shfl_xor_sync(0xffffffffu, Q2[hh], 1); Q2[hh] += __shfl_xor_sync(0xffffffffu, Q2[hh], 2);
    if (tq == 0) s_m[warp * 16 + gq + 8 * hh] = m[hh];
  }
  __syncthreads();
#pragma unroll
  for (int hh = 0; hh < 2; ++hh) {
    const int r = gq + 8 * hh;
    const float M = fmaxf(fmaxf(s_m[r], s_m[16 + r]), fmaxf(s_m[32 + r], s_m[48 + r]));
    const float w = exp2f(m[hh] - M);
    if (tq == 0) { s_l[warp * 16 + r] = L[hh] * w; s_q2[warp * 16 + r] = Q2[hh] * w * w; }
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
      *reinterpret_cast<float2*>(s_o + (warp * 16 + r) * DK + 8 * nt + 2 * tq) = make_float2(O[nt][2 * hh] * w, O[nt][2 * hh + 1] * w);
  }
  __syncthreads();
  for (int i = tid; i < G * DK; i += 128) {
    const int g = i / DK, d = i - g * DK;
    const float s = s_o[g * DK + d] + s_o[(16 + g) * DK + d] + s_o[(32 + g) * DK + d] + s_o[(48 + g) * DK + d];
    const int64_t bh = (int64_t)b * H + kvh * G + g;
    sacc[(bh * n_splits + split) * DK + d] = s;
  }
  if (tid < G) {
    const int g = tid;
    const float M = fmaxf(fmaxf(s_m[g], s_m[16 + g]), fmaxf(s_m[32 + g], s_m[48 + g]));
    const float l = s_l[g] + s_l[16 + g] + s_l[32 + g] + s_l[48 + g];
    const float q2 = s_q2[g] + s_q2[16 + g] + s_q2[32 + g] + s_q2[48 + g];
    const int64_t bh = (int64_t)b * H + kvh * G + g;
    // the merge kernel works with natural-log maxima
    *reinterpret_cast<float4*>(stats + (bh * n_splits + split) * 4) = make_float4(M <= -1e37f ? kNegBig : M * kLn2, l, q2, 0.f);
  }
}

}  // namespace

bool polar_decode_mma_supported(const atma_polar_decode_args& a) {
  const int G = a.H / a.Hkv;
  return (a.dtype == ATMA_BF16 || a.dtype == ATMA_F16) && (a.dk == 128 || a.dk == 64) && G <= 16;
}

int polar_decode_split_mma(const atma_polar_decode_args& a, cudaStream_t st) {
  dim3 grid(a.n_splits, a.Hkv, a.B);
  const int smem = 16 * a.dk * 2 + kStages * 2 * kTileKeys * a.dk * 2;
#define ATMA_LAUNCH(BF, DKK)                                                                                    \
  do {                                                                                                          \
    auto kern = polar_decode_split_mma_kernel<BF, DKK>;                                                         \
    ATMA_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));                \
    kern<<<grid, 128, smem, st>>>((const uint16_t*)a.q, (const uint16_t*)a.k_cache, (const uint16_t*)a.v_cache, \
                                  a.block_tables, a.bt_stride, a.context_lens, a.spg, a.scratch, a.B, a.H,      \
                                  a.Hkv, a.block_size, a.max_blocks, a.num_blocks, a.n_splits, a.window);       \
  } while (0)
  if (a.dtype == ATMA_BF16) { if (a.dk == 128) ATMA_LAUNCH(true, 128); else ATMA_LAUNCH(true, 64); }
  else { if (a.dk == 128) ATMA_LAUNCH(false, 128); else ATMA_LAUNCH(false, 64); }
#undef ATMA_LAUNCH
  return launch_status("polar_decode (split, mma)");
}

}  // namespace atma
