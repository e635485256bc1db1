// Gated-delta chunked scan for 16-bit inputs, d_k = d_v = 128, chunk = 64: tensor-core version.
//
// Same factorisation as the fp32 kernel (gated_delta_scan.cu):
//   per chunk, independent of the state:  -W = -T diag(beta g) K,  U0 = T diag(beta) V,
//       Qg = diag(g) Q,  Kt = diag(g_C/g) K,  Rq = tril((g_p/g_s) q_p.k_s),  T = (I + A)^-1
//   per chunk, on the state S [dk][dv]:    U = U0 - W S;  O = Qg S + Rq U;  S <- g_C S + Kt^T U
// Kernel A (one CTA per chunk) forms K K^T and Q K^T with mma.sync, inverts the four 16x16
// diagonal blocks of the unit lower triangular system in fp32 by substitution, and solves
// (I + A) [-W | U0] = [-beta g K | beta V] block row by block row with mma.sync, feeding each
// solved 16-row block back as an operand from registers; all factors go to scratch as 16-bit tiles
// (U0 transposed, [v][s], the layout the recurrence kernel adds it in).
// The recurrence over the chunks runs on the tcgen05 kernel of gated_delta_scan_sm100.cu.
#include "common.cuh"
#include "mma_sync.cuh"
#include "gated_delta_scan.cuh"

namespace atma {

using namespace mma;
using namespace scan;

namespace {

// ------------------------------------------------------------------------------------------------
// Kernel A: chunk-local factors
// ------------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t a) {
  uint32_t d;
  asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(d) : "r"(a));
  return d;
}

__global__ void varlen_chunk_offsets_kernel(const int32_t* __restrict__ cu_seqlens, int32_t* __restrict__ cu_chunks, int n_seqs) {
  if (threadIdx.x == 0 && blockIdx.x == 0) {
    int acc = 0;
    cu_chunks[0] = 0;
    for (int i = 0; i < n_seqs; ++i) {
      const int len = max(cu_seqlens[i + 1] - cu_seqlens[i], 0);
      acc += (len + kC - 1) / kC;
      cu_chunks[i + 1] = acc;
    }
  }
}

constexpr int kAfLd = 66;      // fp32 A rows: even stride so that column pairs are 8-byte aligned
constexpr int kTfLd = 17;

template <bool kBf16>
__global__ void __launch_bounds__(128, 3)
scan_local_mma_kernel(const uint16_t* __restrict__ q, const uint16_t* __restrict__ k, const uint16_t* __restrict__ v,
                      const float* __restrict__ g, const float* __restrict__ beta, uint8_t* __restrict__ rec_base,
                      float* __restrict__ gc_base, int Tlen, int H, int Hkv, int NC, int normalize_qk, float scale,
                      const VarLen var) {
  extern __shared__ __align__(128) uint8_t sm[];
  uint8_t* Ks = sm;                         // [64][128] 16-bit, swizzled
  uint8_t* Qs = Ks + kC * kD * 2;
  uint8_t* Vs = Qs + kC * kD * 2;
  float* Af = reinterpret_cast<float*>(Vs + kC * kD * 2);      // [64][66] strictly lower triangular A
  float* Tf = Af + kC * kAfLd;                                  // [4][16][17] inverses of the diagonal blocks
  uint8_t* Gb = Qs;                                             // [64][64] 16-bit, swizzled: the solve operator (Q is dead by then)
  float* lg = Tf + 4 * 16 * kTfLd;                              // [64] inclusive log decay
  float* bt = lg + kC;                                          // [64] beta
  float* kinv = bt + kC;                                        // [64]
  float* qinv = kinv + kC;                                      // [64]
  float* wsum = qinv + kC;                                      // [2]

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int c = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  int t0 = c * kC;                          // first token of the chunk on the (b, token) axis
  int rows = min(kC, Tlen - t0);
  if (var.cu_seqlens != nullptr) {          // packed batch: find the sequence that owns chunk c
    if (c >= var.cu_chunks[var.n_seqs]) return;
    int lo_s = 0, hi_s = var.n_seqs;        // largest s with cu_chunks[s] <= c
    while (hi_s - lo_s > 1) {
      const int mid = (lo_s + hi_s) >> 1;
      if (var.cu_chunks[mid] <= c) lo_s = mid; else hi_s = mid;
    }
    t0 = var.cu_seqlens[lo_s] + (c - var.cu_chunks[lo_s]) * kC;
    rows = min(kC, var.cu_seqlens[lo_s + 1] - t0);
  }
  const int hk = h / (H / Hkv);
  uint8_t* rec = rec_base + (((int64_t)b * H + h) * NC + c) * (int64_t)kRecBytes;

  // ---- stage K, Q, V rows (zero beyond the sequence end) -----------------------------------------
  for (int i = tid; i < kC * 16; i += 128) {
    const int r = i >> 4, ch = i & 15;
    const bool ok = r < rows;
    const int64_t tok = (int64_t)b * Tlen + t0 + (ok ? r : 0);
    cp_async16(smem_u32(Ks) + tile_off(r, ch * 8, kD), k + (tok * Hkv + hk) * kD + ch * 8, ok);
    cp_async16(smem_u32(Qs) + tile_off(r, ch * 8, kD), q + (tok * H + h) * kD + ch * 8, ok);
    cp_async16(smem_u32(Vs) + tile_off(r, ch * 8, kD), v + (tok * Hkv + hk) * kD + ch * 8, ok);
  }
  cp_async_commit();
  // inclusive prefix sum of the log decay over the chunk: one row per thread, two warps
  float run = 0.f;
  if (tid < kC) {
    const int64_t gi = ((int64_t)b * Tlen + t0 + tid) * H + h;
    run = (tid < rows) ? g[gi] : 0.f;
    bt[tid] = (tid < rows) ? beta[gi] : 0.f;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const float up = __shfl_up_sync(0xffffffffu, run, o);
      if (lane >= o) run += up;
    }
    if (lane == 31) wsum[warp] = run;
  }
  cp_async_wait<0>();
  __syncthreads();
  if (tid < kC) {
    if (warp == 1) run += wsum[0];
    lg[tid] = run;
    if (tid == kC - 1) gc_base[((int64_t)b * H + h) * NC + c] = __expf(run);
  }

  // ---- row norms: thread i handles row i%64 of K (i < 64) or Q ----------------------------------------
  {
    const int r = tid & 63;
    const uint8_t* src = (tid < 64) ? Ks : Qs;
    float ss = 0.f;
#pragma unroll
    for (int ch = 0; ch < 16; ++ch) {
      const uint4 u = *reinterpret_cast<const uint4*>(src + tile_off(r, ch * 8, kD));
      const uint32_t w4[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) { const float2 f = unpack2<kBf16>(w4[e]); ss = fmaf(f.x, f.x, fmaf(f.y, f.y, ss)); }
    }
    const float inv = normalize_qk ? 1.0f / fmaxf(sqrtf(ss), 1e-12f) : 1.0f;
    if (tid < 64) kinv[r] = inv; else qinv[r] = inv * scale;
  }
  __syncthreads();

  // ---- K K^T for row block `warp` and Q K^T for row block 3 - warp (key blocks at or below the
  //      diagonal only): every warp does five 16x16 block products per k-step ------------------------
  {
    const int rk = warp, rq = 3 - warp;
    float kk[8][4], qk[8][4];
#pragma unroll
    for (int nt = 0; nt < 8; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) { kk[nt][e] = 0.f; qk[nt][e] = 0.f; }
    int am, ak, bn, bk;
    a_rowmajor_lane(lane, am, ak);
    b_nk_lane(lane, bn, bk);
#pragma unroll
    for (int ks = 0; ks < 8; ++ks) {
      uint32_t ak_[4], aq_[4];
      ldsm_x4(smem_u32(Ks) + tile_off(16 * rk + am, 16 * ks + ak, kD), ak_);
      ldsm_x4(smem_u32(Qs) + tile_off(16 * rq + am, 16 * ks + ak, kD), aq_);
#pragma unroll
      for (int pr = 0; pr < 4; ++pr) {
        uint32_t bf[4];
        ldsm_x4(smem_u32(Ks) + tile_off(16 * pr + bn, 16 * ks + bk, kD), bf);
        if (pr <= rk) {
          mma16816<kBf16>(kk[2 * pr], ak_, bf[0], bf[1]);
          mma16816<kBf16>(kk[2 * pr + 1], ak_, bf[2], bf[3]);
        }
        if (pr <= rq) {
          mma16816<kBf16>(qk[2 * pr], aq_, bf[0], bf[1]);
          mma16816<kBf16>(qk[2 * pr + 1], aq_, bf[2], bf[3]);
        }
      }
    }
    // decay ratios, masks; A -> smem fp32, Rq -> scratch (16-bit)
    uint16_t* rq_out = reinterpret_cast<uint16_t*>(rec + kRecRq);
    const int gq = lane >> 2, tq = lane & 3;
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) {
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        {                                                        // A rows of block rk
          const int p = 16 * rk + gq + 8 * half;
          float a2[2];
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const int s = 8 * nt + 2 * tq + e;
            a2[e] = (s < p) ? bt[p] * __expf(lg[p] - lg[s]) * kk[nt][2 * half + e] * kinv[p] * kinv[s] : 0.f;
          }
          *reinterpret_cast<float2*>(Af + p * kAfLd + 8 * nt + 2 * tq) = make_float2(a2[0], a2[1]);
        }
        {                                                        // Rq rows of block rq
          const int p = 16 * rq + gq + 8 * half;
          float r2[2];
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const int s = 8 * nt + 2 * tq + e;
            r2[e] = (s <= p) ? __expf(lg[p] - lg[s]) * qk[nt][2 * half + e] * qinv[p] * kinv[s] : 0.f;
          }
          *reinterpret_cast<uint32_t*>(rq_out + p * kC + 8 * nt + 2 * tq) = pack2<kBf16>(r2[0], r2[1]);
        }
      }
    }
  }
  __syncthreads();

  // ---- emit Qg and Kt; turn K into -beta g K and V into beta V in place (right-hand sides) -------------
  {
    const float lgC = lg[kC - 1];
    uint4* qg_out = reinterpret_cast<uint4*>(rec + kRecQg);
    uint4* kt_out = reinterpret_cast<uint4*>(rec + kRecKt);
    for (int i = tid; i < kC * 16; i += 128) {
      const int r = i >> 4, ch = i & 15;
      const float eg = __expf(lg[r]);
      const float sq = eg * qinv[r], sk = __expf(lgC - lg[r]) * kinv[r];
      const float sbk = -bt[r] * eg * kinv[r], sbv = bt[r];
      uint4 uq = *reinterpret_cast<const uint4*>(Qs + tile_off(r, ch * 8, kD));
      uint4* pk = reinterpret_cast<uint4*>(Ks + tile_off(r, ch * 8, kD));
      uint4* pv = reinterpret_cast<uint4*>(Vs + tile_off(r, ch * 8, kD));
      uint4 uk = *pk, uv = *pv, oq, okt, obk, obv;
      const uint32_t *wq = &uq.x, *wk = &uk.x, *wv = &uv.x;
      uint32_t *xq = &oq.x, *xkt = &okt.x, *xbk = &obk.x, *xbv = &obv.x;
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 fq = unpack2<kBf16>(wq[e]), fk = unpack2<kBf16>(wk[e]), fv = unpack2<kBf16>(wv[e]);
        xq[e] = pack2<kBf16>(fq.x * sq, fq.y * sq);
        xkt[e] = pack2<kBf16>(fk.x * sk, fk.y * sk);
        xbk[e] = pack2<kBf16>(fk.x * sbk, fk.y * sbk);
        xbv[e] = pack2<kBf16>(fv.x * sbv, fv.y * sbv);
      }
      qg_out[i] = oq; kt_out[i] = okt;
      *pk = obk; *pv = obv;
    }
  }

  // ---- inverses of the four 16x16 diagonal blocks of I + A by substitution (fp32) ----------------------
  if (tid < 64) {
    const int blk = tid >> 4, j = tid & 15;
    float x[16];
#pragma unroll
    for (int p = 0; p < 16; ++p) {
      float acc = (p == j) ? 1.f : 0.f;
#pragma unroll
      for (int s = 0; s < p; ++s) acc = fmaf(-Af[(16 * blk + p) * kAfLd + 16 * blk + s], x[s], acc);
      x[p] = acc;
      Tf[(blk * 16 + p) * kTfLd + j] = acc;
    }
  }
  __syncthreads();

  // ---- the solve operator G (16-bit A operand): G_ii = T_ii, G_ij = -T_ii A_ij for j < i ---------------
  //      (I + A) X = R  <=>  X_i = G_ii R_i + sum_{j<i} G_ij X_j, blocks of 16 rows
  {
    // off-diagonal blocks: 6 blocks x 16 rows x 8 column pairs = 768 pairs, 6 per thread
#pragma unroll
    for (int it = 0; it < 6; ++it) {
      const int o = tid + 128 * it;
      const int blk = o >> 7;                                   // 0..5 -> (1,0) (2,0) (2,1) (3,0) (3,1) (3,2)
      const int bi = (blk == 0) ? 1 : (blk < 3 ? 2 : 3);
      const int bj = (blk == 0) ? 0 : (blk < 3 ? blk - 1 : blk - 3);
      const int rr = (o >> 3) & 15, cc = (o & 7) * 2;
      float a0 = 0.f, a1 = 0.f;
#pragma unroll
      for (int s = 0; s < 16; ++s) {
        const float t = Tf[(bi * 16 + rr) * kTfLd + s];
        const float2 a = *reinterpret_cast<const float2*>(Af + (16 * bi + s) * kAfLd + 16 * bj + cc);
        a0 = fmaf(t, a.x, a0); a1 = fmaf(t, a.y, a1);
      }
      *reinterpret_cast<uint32_t*>(Gb + tile_off(16 * bi + rr, 16 * bj + cc, kC)) = pack2<kBf16>(-a0, -a1);
    }
    // diagonal blocks: 4 x 16 x 8 pairs = 512 pairs, 4 per thread
#pragma unroll
    for (int it = 0; it < 4; ++it) {
      const int o = tid + 128 * it;
      const int bi = o >> 7, rr = (o >> 3) & 15, cc = (o & 7) * 2;
      *reinterpret_cast<uint32_t*>(Gb + tile_off(16 * bi + rr, 16 * bi + cc, kC)) =
          pack2<kBf16>(Tf[(bi * 16 + rr) * kTfLd + cc], Tf[(bi * 16 + rr) * kTfLd + cc + 1]);
    }
  }

  __syncthreads();

  // ---- blocked forward solve: -W (warps 0,1) and U0 (warps 2,3), 64 columns per warp.  A solved
  //      block goes back in as a B operand straight from the accumulators (8x8 register transposes),
  //      so the four steps need no barrier ------------------------------------------------------------
  {
    int am, ak, bk, bn;
    a_rowmajor_lane(lane, am, ak);
    b_kn_lane(lane, bk, bn);
    const int gq = lane >> 2, tq = lane & 3;
    const int which = warp >> 1, cb = (warp & 1) * 64;
    const uint8_t* Bs = which ? Vs : Ks;
    uint16_t* out = reinterpret_cast<uint16_t*>(rec + (which ? kRecU0 : kRecW));
    uint32_t xb[3][8][2];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float acc[8][4];
#pragma unroll
      for (int nt = 0; nt < 8; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[nt][e] = 0.f;
      uint32_t af[4];
      ldsm_x4(smem_u32(Gb) + tile_off(16 * i + am, 16 * i + ak, kC), af);
#pragma unroll
      for (int pr = 0; pr < 4; ++pr) {
        uint32_t bf[4];
        ldsm_x4_trans(smem_u32(Bs) + tile_off(16 * i + bk, cb + 16 * pr + bn, kD), bf);
        mma16816<kBf16>(acc[2 * pr], af, bf[0], bf[1]);
        mma16816<kBf16>(acc[2 * pr + 1], af, bf[2], bf[3]);
      }
#pragma unroll
      for (int j = 0; j < 3; ++j) {
        if (j < i) {
          ldsm_x4(smem_u32(Gb) + tile_off(16 * i + am, 16 * j + ak, kC), af);
#pragma unroll
          for (int nt = 0; nt < 8; ++nt) mma16816<kBf16>(acc[nt], af, xb[j][nt][0], xb[j][nt][1]);
        }
      }
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) {
        const uint32_t lo = pack2<kBf16>(acc[nt][0], acc[nt][1]), hi = pack2<kBf16>(acc[nt][2], acc[nt][3]);
        const uint32_t lo_t = movmatrix_trans(lo), hi_t = movmatrix_trans(hi);
        if (which) {                                             // U0 goes out transposed, [v][s]
          *reinterpret_cast<uint32_t*>(out + (cb + 8 * nt + gq) * kC + 16 * i + 2 * tq) = lo_t;
          *reinterpret_cast<uint32_t*>(out + (cb + 8 * nt + gq) * kC + 16 * i + 8 + 2 * tq) = hi_t;
        } else {
          *reinterpret_cast<uint32_t*>(out + (16 * i + gq) * kD + cb + 8 * nt + 2 * tq) = lo;
          *reinterpret_cast<uint32_t*>(out + (16 * i + gq + 8) * kD + cb + 8 * nt + 2 * tq) = hi;
        }
        if (i < 3) { xb[i][nt][0] = lo_t; xb[i][nt][1] = hi_t; }
      }
    }
  }
}

}  // namespace

bool gated_delta_scan_mma_supported(int dtype, int dk, int dv) {
  return (dtype == ATMA_BF16 || dtype == ATMA_F16) && dk == kD && dv == kD;
}

int64_t gated_delta_scan_mma_scratch_bytes(int B, int T, int H) {
  const int64_t NC = (T + kC - 1) / kC;
  return (int64_t)B * H * NC * kRecBytes + (int64_t)B * H * NC * sizeof(float) + 256;
}

static float* gc_array(void* scratch, int B, int H, int NC) {
  uint8_t* recs = static_cast<uint8_t*>(scratch);
  return reinterpret_cast<float*>(recs + (((int64_t)B * H * NC * kRecBytes + 255) / 256) * 256);
}

// Kernel A only: the chunk-local factors of B sequences into `scratch`.
int gated_delta_scan_mma_factors(const void* q, const void* k, const void* v, int dtype, const float* g,
                                 const float* beta, void* scratch, int B, int T, int H, int Hkv, int normalize_qk,
                                 float scale, cudaStream_t st) {
  const int NC = (T + kC - 1) / kC;
  uint8_t* recs = static_cast<uint8_t*>(scratch);
  float* gcs = gc_array(scratch, B, H, NC);
  const int smemA = 3 * kC * kD * 2 + (kC * kAfLd + 4 * 16 * kTfLd) * 4 + (4 * kC + 4) * 4;   // 70.4 KB: three CTAs per SM
  if (dtype == ATMA_BF16) {
    ATMA_CUDA_OK(cudaFuncSetAttribute(scan_local_mma_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, smemA));
    scan_local_mma_kernel<true><<<dim3(NC, H, B), 128, smemA, st>>>((const uint16_t*)q, (const uint16_t*)k, (const uint16_t*)v, g,
                                                                   beta, recs, gcs, T, H, Hkv, NC, normalize_qk, scale, VarLen{});
  } else {
    ATMA_CUDA_OK(cudaFuncSetAttribute(scan_local_mma_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, smemA));
    scan_local_mma_kernel<false><<<dim3(NC, H, B), 128, smemA, st>>>((const uint16_t*)q, (const uint16_t*)k, (const uint16_t*)v, g,
                                                                    beta, recs, gcs, T, H, Hkv, NC, normalize_qk, scale, VarLen{});
  }
  return launch_status("gated_delta_scan (chunk-local, mma)");
}

// Kernel B only: n_rec recurrences over the factors of a scratch built for B sequences.
int gated_delta_scan_mma_recur(void* scratch, int dtype, int B, int T, int H, int n_rec, const int* rec_of,
                               const int* zero_u0, const float* initial_state, void* o, float* final_state,
                               cudaStream_t st) {
  const int NC = (T + kC - 1) / kC;
  if (n_rec < 1 || n_rec > kMaxRec) return fail(ATMA_ERR_INVALID, "gated_delta_scan_recur: n_rec=%d outside 1..%d", n_rec, kMaxRec);
  RecMap map{};
  for (int i = 0; i < n_rec; ++i) {
    map.rec[i] = rec_of ? rec_of[i] : i;
    map.zero_u0[i] = zero_u0 ? zero_u0[i] : 0;
    map.o_row[i] = i;
    if (map.rec[i] < 0 || map.rec[i] >= B)
      return fail(ATMA_ERR_INVALID, "gated_delta_scan_recur: rec_of[%d]=%d outside the %d factor sets", i, map.rec[i], B);
  }
  const uint8_t* recs = static_cast<const uint8_t*>(scratch);
  const float* gcs = gc_array(scratch, B, H, NC);
  return gated_delta_recur_sm100(recs, gcs, dtype == ATMA_BF16, (int64_t)B * H * NC, initial_state, o, final_state, T, H, NC,
                                 n_rec, map, VarLen{}, st);
}

// Packed batch: chunk offsets, factors of every chunk, one recurrence per sequence, all in one go.
// Scratch layout: records of NCu = total/64 + n_seqs chunks per head | g_C | cu_chunks.
int64_t gated_delta_scan_mma_varlen_scratch_bytes(int64_t total_tokens, int n_seqs, int H) {
  const int64_t NCu = total_tokens / kC + n_seqs;
  return gated_delta_scan_mma_scratch_bytes(1, (int)(NCu * kC), H) + (((int64_t)n_seqs + 1) * 4 + 255) / 256 * 256;
}

int gated_delta_scan_mma_varlen(const void* q, const void* k, const void* v, int dtype, const float* g, const float* beta,
                                const int32_t* cu_seqlens, int n_seqs, int64_t total_tokens, const float* initial_state,
                                float* final_state, float* state_table, int64_t slot_stride, const int64_t* slots,
                                const int32_t* has_initial, void* o, void* scratch, int H, int Hkv, int normalize_qk,
                                float scale, float* snapshots, const int32_t* snap_offsets, int snap_chunks,
                                cudaStream_t st) {
  const int NCu = (int)(total_tokens / kC) + n_seqs;          // upper bound on the chunk count
  uint8_t* recs = static_cast<uint8_t*>(scratch);
  float* gcs = gc_array(scratch, 1, H, NCu);
  int32_t* cu_chunks = reinterpret_cast<int32_t*>(recs + gated_delta_scan_mma_scratch_bytes(1, NCu * kC, H));
  varlen_chunk_offsets_kernel<<<1, 32, 0, st>>>(cu_seqlens, cu_chunks, n_seqs);
  VarLen var{cu_seqlens, cu_chunks, n_seqs, slots, has_initial, state_table, slot_stride, snapshots, snap_offsets, snap_chunks};
  const int smemA = 3 * kC * kD * 2 + (kC * kAfLd + 4 * 16 * kTfLd) * 4 + (4 * kC + 4) * 4;   // 70.4 KB: three CTAs per SM
  const bool bf = dtype == ATMA_BF16;
  if (bf) {
    ATMA_CUDA_OK(cudaFuncSetAttribute(scan_local_mma_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, smemA));
    scan_local_mma_kernel<true><<<dim3(NCu, H, 1), 128, smemA, st>>>((const uint16_t*)q, (const uint16_t*)k, (const uint16_t*)v, g,
                                                                    beta, recs, gcs, 0, H, Hkv, NCu, normalize_qk, scale, var);
  } else {
    ATMA_CUDA_OK(cudaFuncSetAttribute(scan_local_mma_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, smemA));
    scan_local_mma_kernel<false><<<dim3(NCu, H, 1), 128, smemA, st>>>((const uint16_t*)q, (const uint16_t*)k, (const uint16_t*)v, g,
                                                                     beta, recs, gcs, 0, H, Hkv, NCu, normalize_qk, scale, var);
  }
  int rc = launch_status("gated_delta_scan (packed, chunk-local, mma)");
  if (rc != ATMA_OK) return rc;
  return gated_delta_recur_sm100(recs, gcs, bf, (int64_t)H * NCu, initial_state, o, final_state, 0, H, NCu, n_seqs, RecMap{}, var,
                                 st);
}

int gated_delta_scan_mma(const void* q, const void* k, const void* v, int dtype, const float* g, const float* beta,
                         const float* initial_state, void* o, float* final_state, void* scratch, int B, int T, int H,
                         int Hkv, int normalize_qk, float scale, cudaStream_t st) {
  int rc = gated_delta_scan_mma_factors(q, k, v, dtype, g, beta, scratch, B, T, H, Hkv, normalize_qk, scale, st);
  if (rc != ATMA_OK) return rc;
  int done = 0;
  while (done < B) {                                  // at most kMaxRec recurrences per launch
    const int n = (B - done) < kMaxRec ? (B - done) : kMaxRec;
    int rec_of[kMaxRec];
    for (int i = 0; i < n; ++i) rec_of[i] = done + i;
    const int64_t so = (int64_t)done * H * kD * kD, oo = (int64_t)done * T * H * kD;
    rc = gated_delta_scan_mma_recur(scratch, dtype, B, T, H, n, rec_of, nullptr,
                                    initial_state ? initial_state + so : nullptr,
                                    o ? (void*)((uint16_t*)o + oo) : nullptr, final_state ? final_state + so : nullptr, st);
    if (rc != ATMA_OK) return rc;
    done += n;
  }
  return ATMA_OK;
}

}  // namespace atma
