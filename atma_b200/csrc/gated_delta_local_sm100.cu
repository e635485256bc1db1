// Gated-delta scan, the chunk-local (state-independent) stage, on the 5th-generation tensor cores
// (sm_100a): K, Q, V tiles by TMA, the dense contractions on tcgen05.mma with TMEM accumulators,
// the 64 x 64 unit-lower-triangular inverse per chunk in fp32 / tf32 by the worker warps.
//
// A persistent CTA walks over tiles of TWO 64-token chunks of one head (128 rows, rows 0-63 = the
// first chunk, 64-127 = the second; the two chunks only share the MMA shapes, every product that
// couples them is masked).  Per tile, with g the inclusive decay prefix inside a chunk, k^ and q^
// the L2-normalised rows:
//
//   MMA    Gkk = K K^T,  Gqk = Q K^T                               128 x 128 x 128 each (SS)
//   warps  A[p][s] = beta_p (g_p/g_s) k^_p.k^_s  (s < p)           fp32, shared memory
//          Rq[p][s] = (g_p/g_s) q^_p.k^_s        (s <= p)          -> record
//          Qg = diag(g q_inv) Q,  Kt = diag(g_C/g k_inv) K         -> record
//          T = (I + A)^-1: 16 x 16 diagonal blocks by substitution (fp32), then the blocks below
//          the diagonal level by level with mma.sync tf32 (G_il = -T_ii A_il; T_ij = sum_l G_il T_lj)
//          Tw[p][s] = -T[p][s] beta_s g_s k_inv_s,  Tu[p][s] = T[p][s] beta_s    16-bit tiles
//   MMA    -W = Tw K (B = the K tile itself, MN-major),  U0^T = V^T Tu^T (A = the V tile, MN-major)
//   warps  -W rows and U0^T rows: TMEM -> 16-bit -> record
//
// Folding the row scalings of the right-hand sides into the columns of T leaves the K and V tiles
// untouched in shared memory, so they serve as MMA operands exactly as TMA delivered them.
//
//   warp 0      TMA producer        warp 1      MMA issuer (one lane); owns the TMEM allocation
//   warps 2-9   workers; warp w works on TMEM lanes / tile rows 32 (w % 4) .. +31 and on column
//               half (w - 2) / 4 of whatever it reads
// TMEM (512 columns): Gkk [0,128) Gqk [128,256) -W [256,384) U0^T [384,512).
// Every mbarrier wait is bounded; on expiry the CTA frees its TMEM, returns and leaves a status
// word for the host.
#include "common.cuh"
#include "sm100.cuh"
#include "gated_delta_scan.cuh"

namespace atma {

using namespace sm100;
using namespace scan;

namespace {

__device__ int g_local_status = 0;

constexpr int kThreads = 320;                     // TMA warp, MMA warp, eight worker warps
constexpr int kTile = 2 * kD * 128;               // a [128][128] 16-bit tile = two 64-column boxes of 16 KiB
constexpr int kLd = 68;                           // fp32 row stride of the A and T matrices
constexpr int kOffK = 0, kOffQ = kTile, kOffV = 2 * kTile, kOffTu = 3 * kTile, kOffAf = 4 * kTile,
              kOffTf = kOffAf + 128 * kLd * 4, kSmemBytes = kOffTf + 128 * kLd * 4 + 1024;
constexpr uint32_t kColKK = 0, kColQK = 128, kColW = 256, kColU = 384;

struct Barriers { uint64_t kq_full, v_full, g_done, t_ready, wu_done; };

struct Meta { int64_t t0[2]; int rows[2]; int64_t rec[2]; int h, hk; };

struct Params {
  const float* g; const float* beta;
  uint8_t* recs; float* gcs;
  int Tlen, H, Hkv, NC, B, normalize;
  float scale;
  int n_pairs; int64_t n_tiles;
  VarLen var;
};

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
  if constexpr (kBf16) return make_float2(__uint_as_float(v << 16), __uint_as_float(v & 0xffff0000u));
  else return __half22float2(*reinterpret_cast<__half2*>(&v));
}
__device__ __forceinline__ uint32_t box_off(int row, int chunk) {
  return (uint32_t)(row * 128 + ((chunk ^ (row & 7)) << 4));
}
__device__ __forceinline__ void worker_sync() { asm volatile("bar.sync 1, 256;" ::: "memory"); }

__device__ __forceinline__ void mma_tf32(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// acc (16 x 16 as two 8-column tiles) += A (16 x 16, row-major, stride kLd) * B (16 x 16, row-major, stride kLd)
__device__ __forceinline__ void block_mma(float (&acc)[2][4], const float* A, const float* Bm, int lane) {
  const int g = lane >> 2, t = lane & 3;
#pragma unroll
  for (int ks = 0; ks < 2; ++ks) {
    uint32_t a[4];
    a[0] = __float_as_uint(A[g * kLd + 8 * ks + t]);
    a[1] = __float_as_uint(A[(g + 8) * kLd + 8 * ks + t]);
    a[2] = __float_as_uint(A[g * kLd + 8 * ks + t + 4]);
    a[3] = __float_as_uint(A[(g + 8) * kLd + 8 * ks + t + 4]);
#pragma unroll
    for (int nt = 0; nt < 2; ++nt)
      mma_tf32(acc[nt], a, __float_as_uint(Bm[(8 * ks + t) * kLd + 8 * nt + g]), __float_as_uint(Bm[(8 * ks + t + 4) * kLd + 8 * nt + g]));
  }
}
__device__ __forceinline__ void block_store(float* C, const float (&acc)[2][4], int lane, float sign) {
  const int g = lane >> 2, t = lane & 3;
#pragma unroll
  for (int nt = 0; nt < 2; ++nt) {
    *reinterpret_cast<float2*>(C + g * kLd + 8 * nt + 2 * t) = make_float2(sign * acc[nt][0], sign * acc[nt][1]);
    *reinterpret_cast<float2*>(C + (g + 8) * kLd + 8 * nt + 2 * t) = make_float2(sign * acc[nt][2], sign * acc[nt][3]);
  }
}

__device__ __forceinline__ void tile_meta(const Params& p, int64_t tile, Meta& m) {
  m.h = (int)(tile % p.H);
  m.hk = m.h / (p.H / p.Hkv);
  const int64_t rest = tile / p.H;
  const int j = (int)(rest % p.n_pairs);
  const int b = (int)(rest / p.n_pairs);
#pragma unroll
  for (int ci = 0; ci < 2; ++ci) {
    const int c = 2 * j + ci;
    m.t0[ci] = 0; m.rows[ci] = 0; m.rec[ci] = -1;
    if (p.var.cu_seqlens != nullptr) {
      const int total = p.var.cu_chunks[p.var.n_seqs];
      if (c < total) {
        int lo = 0, hi = p.var.n_seqs;                // largest s with cu_chunks[s] <= c
        while (hi - lo > 1) {
          const int mid = (lo + hi) >> 1;
          if (p.var.cu_chunks[mid] <= c) lo = mid; else hi = mid;
        }
        m.t0[ci] = (int64_t)p.var.cu_seqlens[lo] + (int64_t)(c - p.var.cu_chunks[lo]) * kC;
        m.rows[ci] = (int)min((int64_t)kC, (int64_t)p.var.cu_seqlens[lo + 1] - m.t0[ci]);
        m.rec[ci] = (int64_t)m.h * p.NC + c;
      }
    } else if (c < p.NC) {
      m.t0[ci] = (int64_t)b * p.Tlen + (int64_t)c * kC;
      m.rows[ci] = min(kC, p.Tlen - c * kC);
      m.rec[ci] = ((int64_t)b * p.H + m.h) * p.NC + c;
    }
  }
}

template <bool kBf16>
__global__ void __launch_bounds__(kThreads, 1)
scan_local_sm100_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                        const __grid_constant__ CUtensorMap tmap_v, const Params p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* Ks = smem + kOffK;
  uint8_t* Qs = smem + kOffQ;                       // the Q tile, later the Tw tile
  uint8_t* Vs = smem + kOffV;
  uint8_t* Tus = smem + kOffTu;
  float* Af = reinterpret_cast<float*>(smem + kOffAf);
  float* Tf = reinterpret_cast<float*>(smem + kOffTf);
  __shared__ Barriers bar;
  __shared__ uint32_t s_tmem_base;
  __shared__ int s_abort;
  __shared__ float s_lg[128], s_bt[128], s_kinv[128], s_qsc[128], s_ksc[128], s_wsc[128], s_part[4][128], s_wsum[4];

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid == 0) {
    mbar_init(&bar.kq_full, 1); mbar_init(&bar.v_full, 1); mbar_init(&bar.g_done, 1);
    mbar_init(&bar.t_ready, 8); mbar_init(&bar.wu_done, 1);
    s_abort = 0;
    fence_barrier_init();
  }
  if (warp == 1) tmem_alloc(&s_tmem_base, 512);
  if (warp == 0 && lane == 0) { prefetch_tensormap(&tmap_q); prefetch_tensormap(&tmap_k); prefetch_tensormap(&tmap_v); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tbase = s_tmem_base;
  volatile int* abort_flag = &s_abort;

  if (warp == 0) {
    // =============================== TMA producer ================================================
    if (lane == 0) {
      uint32_t it = 0;
      for (int64_t tile = blockIdx.x; tile < p.n_tiles; tile += gridDim.x, ++it) {
        // the K, Q (by then Tw) and V tiles are dead as soon as the previous tile's last products are done
        if (it > 0 && !mbar_wait(&bar.wu_done, (it - 1) & 1u, abort_flag)) break;
        Meta m;
        tile_meta(p, tile, m);
        mbar_arrive_expect_tx(&bar.kq_full, 2 * kTile);
#pragma unroll
        for (int ci = 0; ci < 2; ++ci)
#pragma unroll
          for (int cb = 0; cb < 2; ++cb) {
            tma_load_4d(Ks + cb * 16384 + ci * 8192, &tmap_k, &bar.kq_full, cb * 64, m.hk, (int)(ci ? m.t0[1] : m.t0[0]), 0);
            tma_load_4d(Qs + cb * 16384 + ci * 8192, &tmap_q, &bar.kq_full, cb * 64, m.h, (int)(ci ? m.t0[1] : m.t0[0]), 0);
          }
        mbar_arrive_expect_tx(&bar.v_full, kTile);
#pragma unroll
        for (int ci = 0; ci < 2; ++ci)
#pragma unroll
          for (int cb = 0; cb < 2; ++cb)
            tma_load_4d(Vs + cb * 16384 + ci * 8192, &tmap_v, &bar.v_full, cb * 64, m.hk, (int)(ci ? m.t0[1] : m.t0[0]), 0);
        // the shared-memory tiles stay busy until this tile's last products; meanwhile bring the next tile's
        // inputs into L2, so that its loads do not wait for DRAM
        if (tile + gridDim.x < p.n_tiles) {
          Meta mn;
          tile_meta(p, tile + gridDim.x, mn);
#pragma unroll
          for (int ci = 0; ci < 2; ++ci)
#pragma unroll
            for (int cb = 0; cb < 2; ++cb) {
              tma_prefetch_l2_4d(&tmap_k, cb * 64, mn.hk, (int)mn.t0[ci], 0);
              tma_prefetch_l2_4d(&tmap_q, cb * 64, mn.h, (int)mn.t0[ci], 0);
              tma_prefetch_l2_4d(&tmap_v, cb * 64, mn.hk, (int)mn.t0[ci], 0);
            }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // =============================== MMA issuer =================================================
    if (lane == 0) {
      constexpr int fmt = kBf16 ? 1 : 0;
      constexpr uint32_t idesc_kk = make_idesc(128, 128, fmt, 0, 0);     // both operands K-major
      constexpr uint32_t idesc_w = make_idesc(128, 128, fmt, 0, 1);      // -W = Tw K: B = K tile [s][k], MN-major
      constexpr uint32_t idesc_u = make_idesc(128, 128, fmt, 1, 0);      // U0^T = V^T Tu^T: A = V tile [s][v], MN-major
      const uint64_t hi_k = (uint64_t(1024 >> 4) << 32) | (uint64_t(1) << 46) | (uint64_t(2) << 61) | (uint64_t(16 >> 4) << 16);
      const uint64_t hi_mn = (uint64_t(1024 >> 4) << 32) | (uint64_t(1) << 46) | (uint64_t(2) << 61) | (uint64_t(16384 >> 4) << 16);
      const uint64_t kd = hi_k | uint64_t((smem_u32(Ks) >> 4) & 0x3FFFu), qd = hi_k | uint64_t((smem_u32(Qs) >> 4) & 0x3FFFu);
      const uint64_t tud = hi_k | uint64_t((smem_u32(Tus) >> 4) & 0x3FFFu);
      const uint64_t kmn = hi_mn | uint64_t((smem_u32(Ks) >> 4) & 0x3FFFu), vmn = hi_mn | uint64_t((smem_u32(Vs) >> 4) & 0x3FFFu);
      uint32_t it = 0;
      bool ok = true;
      for (int64_t tile = blockIdx.x; tile < p.n_tiles && ok; tile += gridDim.x, ++it) {
        ok = mbar_wait(&bar.kq_full, it & 1u, abort_flag);
        if (!ok) break;
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          const uint64_t off = uint64_t(((kk >> 2) * 16384 + (kk & 3) * 32) >> 4);
          mma_ss(tbase + kColKK, kd + off, kd + off, idesc_kk, kk > 0);
        }
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          const uint64_t off = uint64_t(((kk >> 2) * 16384 + (kk & 3) * 32) >> 4);
          mma_ss(tbase + kColQK, qd + off, kd + off, idesc_kk, kk > 0);
        }
        tc_commit(&bar.g_done);
        ok = mbar_wait(&bar.t_ready, it & 1u, abort_flag);
        if (ok) ok = mbar_wait(&bar.v_full, it & 1u, abort_flag);
        if (!ok) break;
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {                 // A = Tw (in the Q tile's place), K-major over s
          const uint64_t off = uint64_t(((kk >> 2) * 16384 + (kk & 3) * 32) >> 4);
          mma_ss(tbase + kColW, qd + off, kmn + uint64_t((kk * 2048) >> 4), idesc_w, kk > 0);
        }
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          const uint64_t off = uint64_t(((kk >> 2) * 16384 + (kk & 3) * 32) >> 4);
          mma_ss(tbase + kColU, vmn + uint64_t((kk * 2048) >> 4), tud + off, idesc_u, kk > 0);
        }
        tc_commit(&bar.wu_done);
      }
    }
    __syncwarp();
  } else {
    // =============================== workers ====================================================
    const int wtid = tid - 64;
    const int quad = warp & 3, half = (warp - 2) >> 2;
    const int row = 32 * quad + lane;                  // tile row p (and TMEM lane)
    const int ci = row >> 6, pr = row & 63;            // chunk of the tile, row inside the chunk
    const uint32_t lane_base = tbase + (uint32_t(32 * quad) << 16);
    uint32_t it = 0;
    bool ok = true;
    // the tile's coordinates, and g and beta of this thread's row (first column half only), are
    // fetched one tile ahead, in the shadow of the wait for the previous tile's last products
    Meta m_next{};
    float g_pre = 0.f, b_pre = 0.f;
    auto prefetch_tile = [&](int64_t tile) {
      if (tile < p.n_tiles) {
        tile_meta(p, tile, m_next);
        if (half == 0) {
          const bool v = pr < (ci ? m_next.rows[1] : m_next.rows[0]);
          const int64_t gi = ((ci ? m_next.t0[1] : m_next.t0[0]) + pr) * p.H + m_next.h;
          g_pre = v ? p.g[gi] : 0.f;
          b_pre = v ? p.beta[gi] : 0.f;
        }
      }
    };
    prefetch_tile(blockIdx.x);
    for (int64_t tile = blockIdx.x; tile < p.n_tiles; tile += gridDim.x, ++it) {
      const Meta m = m_next;
      const bool valid = pr < (ci ? m.rows[1] : m.rows[0]);
      const bool have = (ci ? m.rec[1] : m.rec[0]) >= 0;

      worker_sync();                                     // every warp is done with the previous tile's arrays
      // ---- decay prefix and beta: one row per thread of the first column half ---------------------
      float run = 0.f;
      if (half == 0) {
        run = g_pre;
        s_bt[row] = b_pre;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
          const float up = __shfl_up_sync(0xffffffffu, run, o);
          if (lane >= o) run += up;
        }
        if (lane == 31) s_wsum[quad] = run;
      }
      // ---- row norms of K and Q: each thread sums its 64 columns --------------------------------------
      ok = mbar_wait(&bar.kq_full, it & 1u, abort_flag);
      (void)ok;                                            // after a timeout every later wait returns at once; the
                                                           // warps keep walking the same barriers
      {
        float sk = 0.f, sq = 0.f;
#pragma unroll
        for (int ch = 0; ch < 8; ++ch) {
          const uint4 uk = *reinterpret_cast<const uint4*>(Ks + half * 16384 + box_off(row, ch));
          const uint4 uq = *reinterpret_cast<const uint4*>(Qs + half * 16384 + box_off(row, ch));
          const uint32_t wk[4] = {uk.x, uk.y, uk.z, uk.w}, wq[4] = {uq.x, uq.y, uq.z, uq.w};
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float2 fk = unpack2<kBf16>(wk[e]), fq = unpack2<kBf16>(wq[e]);
            sk = fmaf(fk.x, fk.x, fmaf(fk.y, fk.y, sk));
            sq = fmaf(fq.x, fq.x, fmaf(fq.y, fq.y, sq));
          }
        }
        s_part[half][row] = sk;
        s_part[2 + half][row] = sq;
      }
      worker_sync();
      const float kinv_p = p.normalize ? 1.0f / fmaxf(sqrtf(s_part[0][row] + s_part[1][row]), 1e-12f) : 1.0f;
      const float qinv_p = (p.normalize ? 1.0f / fmaxf(sqrtf(s_part[2][row] + s_part[3][row]), 1e-12f) : 1.0f) * p.scale;
      if (half == 0) {
        if (quad & 1) run += s_wsum[quad - 1];           // second warp of the chunk
        s_lg[row] = run;
        s_kinv[row] = kinv_p;
        if (pr == kC - 1 && have) p.gcs[(ci ? m.rec[1] : m.rec[0])] = __expf(run);
      }
      worker_sync();
      const float lg_p = s_lg[row], bt_p = s_bt[row], lg_C = s_lg[64 * ci + 63];
      if (half == 0) {
        s_qsc[row] = valid ? __expf(lg_p) * qinv_p : 0.f;
        s_ksc[row] = valid ? __expf(lg_C - lg_p) * kinv_p : 0.f;
        s_wsc[row] = -bt_p * __expf(lg_p) * kinv_p;       // column scale of Tw
      }
      worker_sync();

      // ---- Qg and Kt -> record: 16 threads per 256-byte row, so every store instruction of a warp
      //      covers 512 contiguous bytes of the record
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int r = (wtid >> 4) + 16 * i, ch = wtid & 15, rc = r >> 6;
        if ((rc ? m.rec[1] : m.rec[0]) >= 0) {
          uint8_t* rrec = p.recs + (rc ? m.rec[1] : m.rec[0]) * (int64_t)kRecBytes;
          const float sq = s_qsc[r], sk = s_ksc[r];
          const uint4 uk = *reinterpret_cast<const uint4*>(Ks + (ch >> 3) * 16384 + box_off(r, ch & 7));
          const uint4 uq = *reinterpret_cast<const uint4*>(Qs + (ch >> 3) * 16384 + box_off(r, ch & 7));
          const uint32_t wk[4] = {uk.x, uk.y, uk.z, uk.w}, wq[4] = {uq.x, uq.y, uq.z, uq.w};
          uint32_t ok_[4], oq_[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float2 fk = unpack2<kBf16>(wk[e]), fq = unpack2<kBf16>(wq[e]);
            ok_[e] = pack2<kBf16>(fk.x * sk, fk.y * sk);
            oq_[e] = pack2<kBf16>(fq.x * sq, fq.y * sq);
          }
          *reinterpret_cast<uint4*>(rrec + kRecQg + (r & 63) * 256 + ch * 16) = make_uint4(oq_[0], oq_[1], oq_[2], oq_[3]);
          *reinterpret_cast<uint4*>(rrec + kRecKt + (r & 63) * 256 + ch * 16) = make_uint4(ok_[0], ok_[1], ok_[2], ok_[3]);
        }
      }

      // ---- A (fp32, shared memory) and Rq (record) from the Gram matrices -------------------------------
      ok = mbar_wait(&bar.g_done, it & 1u, abort_flag);
      (void)ok;                                            // after a timeout every later wait returns at once; the
                                                           // warps keep walking the same barriers
      tc_fence_after();
      {
        uint32_t gk[32], gq[32];
        uint32_t rq[16];
        // rows 0-31 of a chunk see no column of its second half: that warp only writes zeros
        const bool masked = half == 1 && (quad & 1) == 0;
        if (masked) {
#pragma unroll
          for (int j = 0; j < 32; j += 4) *reinterpret_cast<float4*>(Af + row * kLd + 32 + j) = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
          for (int j = 0; j < 16; ++j) rq[j] = 0u;
        } else {
        tmem_ld32_nowait(lane_base + kColKK + 64 * ci + 32 * half, gk);
        tmem_ld32_nowait(lane_base + kColQK + 64 * ci + 32 * half, gq);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; j += 2) {
          float a2[2], r2[2];
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            reg_fence(gk[j + e]); reg_fence(gq[j + e]);
            const int s = 32 * half + j + e;
            const float dec = __expf(lg_p - s_lg[64 * ci + s]) * s_kinv[64 * ci + s];
            a2[e] = (s < pr) ? bt_p * dec * kinv_p * __uint_as_float(gk[j + e]) : 0.f;
            r2[e] = (s <= pr) ? dec * qinv_p * __uint_as_float(gq[j + e]) : 0.f;
          }
          *reinterpret_cast<float2*>(Af + row * kLd + 32 * half + j) = make_float2(a2[0], a2[1]);
          rq[j >> 1] = pack2<kBf16>(r2[0], r2[1]);
        }
        }
        // staged in the (still unused) Tu tile: [128 rows][8 chunks of 16 bytes], chunk index xor (row & 7)
#pragma unroll
        for (int c4 = 0; c4 < 4; ++c4)
          *reinterpret_cast<uint4*>(Tus + box_off(row, 4 * half + c4)) = make_uint4(rq[4 * c4], rq[4 * c4 + 1], rq[4 * c4 + 2], rq[4 * c4 + 3]);
      }
      worker_sync();
#pragma unroll
      for (int i = 0; i < 4; ++i) {                      // 16 KiB out, 512 contiguous bytes per warp instruction
        const int idx = wtid + 256 * i, r = idx >> 3, ch = idx & 7, rc = r >> 6;
        if ((rc ? m.rec[1] : m.rec[0]) >= 0)
          *reinterpret_cast<uint4*>(p.recs + (rc ? m.rec[1] : m.rec[0]) * (int64_t)kRecBytes + kRecRq + (r & 63) * 128 + ch * 16) =
              *reinterpret_cast<const uint4*>(Tus + box_off(r, ch));
      }

      // ---- T = (I + A)^-1 per chunk: diagonal 16 x 16 blocks by substitution ----------------------------
      if (wtid < 128) {
        const int cc = wtid >> 6, blk = (wtid >> 4) & 3, j = wtid & 15;
        const float* Ab = Af + (64 * cc + 16 * blk) * kLd + 16 * blk;
        float* Tb = Tf + (64 * cc + 16 * blk) * kLd + 16 * blk;
        float x[16];
#pragma unroll
        for (int r = 0; r < 16; ++r) {
          float acc = (r == j) ? 1.f : 0.f;
#pragma unroll
          for (int s = 0; s < r; ++s) acc = fmaf(-Ab[r * kLd + s], x[s], acc);
          x[r] = acc;
          Tb[r * kLd + j] = acc;
        }
      }
      worker_sync();
      // G_il = -T_ii A_il for the six blocks below the diagonal of each chunk (in place over A_il)
      for (int blk = warp - 2; blk < 12; blk += 8) {
        const int cc = blk / 6, e = blk % 6;
        const int bi = (e == 0) ? 1 : (e < 3 ? 2 : 3), bl = (e == 0) ? 0 : (e < 3 ? e - 1 : e - 3);
        float acc[2][4] = {};
        float* Ail = Af + (64 * cc + 16 * bi) * kLd + 16 * bl;
        block_mma(acc, Tf + (64 * cc + 16 * bi) * kLd + 16 * bi, Ail, lane);
        __syncwarp();
        block_store(Ail, acc, lane, -1.f);
      }
      worker_sync();
      // T_ij = sum_{l=j}^{i-1} G_il T_lj, one level of blocks below the diagonal at a time
#pragma unroll 1
      for (int d = 1; d <= 3; ++d) {
        const int per = 4 - d;                          // blocks of this level per chunk
        for (int blk = warp - 2; blk < 2 * per; blk += 8) {
          const int cc = blk / per, bj = blk % per, bi = bj + d;
          float acc[2][4] = {};
          for (int l = bj; l < bi; ++l)
            block_mma(acc, Af + (64 * cc + 16 * bi) * kLd + 16 * l, Tf + (64 * cc + 16 * l) * kLd + 16 * bj, lane);
          block_store(Tf + (64 * cc + 16 * bi) * kLd + 16 * bj, acc, lane, 1.f);
        }
        worker_sync();
      }

      // ---- Tw (over the Q tile) and Tu: this thread's row, 32 columns of its own chunk; zeros in the other chunk's box
      {
        uint8_t* tw_row = Qs + ci * 16384;
        uint8_t* tu_row = Tus + ci * 16384;
        uint8_t* tw_zero = Qs + (1 - ci) * 16384;
        uint8_t* tu_zero = Tus + (1 - ci) * 16384;
#pragma unroll
        for (int c4 = 0; c4 < 4; ++c4) {
          uint32_t w4[4], u4[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            float tw[2], tu[2];
#pragma unroll
            for (int f = 0; f < 2; ++f) {
              const int s = 32 * half + 8 * c4 + 2 * e + f;
              const int bs = s >> 4, bp = pr >> 4;
              float t = 0.f;
              if (bs < bp || (bs == bp && s <= pr)) t = Tf[row * kLd + s];
              tu[f] = t * s_bt[64 * ci + s];
              tw[f] = t * s_wsc[64 * ci + s];
            }
            w4[e] = pack2<kBf16>(tw[0], tw[1]);
            u4[e] = pack2<kBf16>(tu[0], tu[1]);
          }
          const uint32_t off = box_off(row, 4 * half + c4);
          *reinterpret_cast<uint4*>(tw_row + off) = make_uint4(w4[0], w4[1], w4[2], w4[3]);
          *reinterpret_cast<uint4*>(tu_row + off) = make_uint4(u4[0], u4[1], u4[2], u4[3]);
          *reinterpret_cast<uint4*>(tw_zero + off) = make_uint4(0u, 0u, 0u, 0u);
          *reinterpret_cast<uint4*>(tu_zero + off) = make_uint4(0u, 0u, 0u, 0u);
        }
      }
      fence_proxy_async();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bar.t_ready);
      prefetch_tile(tile + gridDim.x);

      // ---- -W rows and U0^T rows: TMEM -> 16-bit -> record ------------------------------------------------
      ok = mbar_wait(&bar.wu_done, it & 1u, abort_flag);
      (void)ok;                                            // after a timeout every later wait returns at once; the
                                                           // warps keep walking the same barriers
      tc_fence_after();
      {
        // staged as [128 rows][16 chunks of 16 bytes] (chunk index xor (row & 7)): -W in the Tu tile, U0^T rows
        // (two 128-byte halves, one per chunk) in the A matrix's space; both are dead until the next tile
        uint8_t* stage_w = Tus;
        uint8_t* stage_u = smem + kOffAf;
        uint32_t r[64];
        tmem_ld32_nowait(lane_base + kColW + 64 * half, &r[0]);
        tmem_ld32_nowait(lane_base + kColW + 64 * half + 32, &r[32]);
        tmem_ld_wait();
#pragma unroll
        for (int ch = 0; ch < 8; ++ch) {
          uint32_t w[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            reg_fence(r[8 * ch + 2 * e]); reg_fence(r[8 * ch + 2 * e + 1]);
            w[e] = pack2<kBf16>(__uint_as_float(r[8 * ch + 2 * e]), __uint_as_float(r[8 * ch + 2 * e + 1]));
          }
          *reinterpret_cast<uint4*>(stage_w + row * 256 + (((8 * half + ch) ^ (row & 7)) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
        }
        // U0^T: lane = value channel v, columns 64*half .. +63 = the rows of chunk `half`
        tmem_ld32_nowait(lane_base + kColU + 64 * half, &r[0]);
        tmem_ld32_nowait(lane_base + kColU + 64 * half + 32, &r[32]);
        tmem_ld_wait();
#pragma unroll
        for (int ch = 0; ch < 8; ++ch) {
          uint32_t w[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            reg_fence(r[8 * ch + 2 * e]); reg_fence(r[8 * ch + 2 * e + 1]);
            w[e] = pack2<kBf16>(__uint_as_float(r[8 * ch + 2 * e]), __uint_as_float(r[8 * ch + 2 * e + 1]));
          }
          *reinterpret_cast<uint4*>(stage_u + half * 16384 + box_off(row, ch)) = make_uint4(w[0], w[1], w[2], w[3]);
        }
        tc_fence_before();
        worker_sync();
#pragma unroll
        for (int i = 0; i < 8; ++i) {                    // -W: 32 KiB out
          const int idx = wtid + 256 * i, r2 = idx >> 4, ch = idx & 15, rc = r2 >> 6;
          if ((rc ? m.rec[1] : m.rec[0]) >= 0)
            *reinterpret_cast<uint4*>(p.recs + (rc ? m.rec[1] : m.rec[0]) * (int64_t)kRecBytes + kRecW + (r2 & 63) * 256 + ch * 16) =
                *reinterpret_cast<const uint4*>(stage_w + r2 * 256 + ((ch ^ (r2 & 7)) << 4));
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) {                    // U0^T of both chunks: 2 x 16 KiB out
          const int idx = wtid + 256 * i, rc = idx >> 10, v = (idx >> 3) & 127, ch = idx & 7;
          if ((rc ? m.rec[1] : m.rec[0]) >= 0)
            *reinterpret_cast<uint4*>(p.recs + (rc ? m.rec[1] : m.rec[0]) * (int64_t)kRecBytes + kRecU0 + v * 128 + ch * 16) =
                *reinterpret_cast<const uint4*>(stage_u + rc * 16384 + box_off(v, ch));
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (tid == 0 && s_abort) atomicExch(&g_local_status, 1);
  if (warp == 1) tmem_dealloc(tbase, 512);
}

// (d, head, token) view of a (tokens, heads, 128) 16-bit tensor; boxes of 64 channels x 64 tokens of one head
int make_input_map(CUtensorMap* out, const void* base, int is_bf16, int heads, int64_t tokens) {
  const uint64_t dims[4] = {128, (uint64_t)heads, (uint64_t)tokens, 1};
  const int64_t strides[3] = {128, (int64_t)heads * 128, (int64_t)heads * 128 * tokens};
  const uint32_t box[4] = {64, 1, 64, 1};
  return make_tmap_16bit_4d(out, base, is_bf16, dims, strides, box);
}

}  // namespace

int gated_delta_local_sm100(const void* q, const void* k, const void* v, int is_bf16, const float* g, const float* beta,
                            uint8_t* recs, float* gcs, int B, int Tlen, int H, int Hkv, int NC, int normalize_qk, float scale,
                            const VarLen& var, int64_t total_tokens, cudaStream_t st) {
  if (NC <= 0 || total_tokens <= 0) return ATMA_OK;
  if (total_tokens >= (int64_t(1) << 31)) return fail(ATMA_ERR_INVALID, "gated_delta_scan: %lld tokens exceed the tensor-map range", (long long)total_tokens);
  CUtensorMap mq, mk, mv;
  int rc = make_input_map(&mq, q, is_bf16, H, total_tokens);
  if (rc == ATMA_OK) rc = make_input_map(&mk, k, is_bf16, Hkv, total_tokens);
  if (rc == ATMA_OK) rc = make_input_map(&mv, v, is_bf16, Hkv, total_tokens);
  if (rc != ATMA_OK) return rc;
  Params p{};
  p.g = g; p.beta = beta; p.recs = recs; p.gcs = gcs;
  p.Tlen = Tlen; p.H = H; p.Hkv = Hkv; p.NC = NC; p.B = B; p.normalize = normalize_qk; p.scale = scale;
  p.n_pairs = (NC + 1) / 2;
  p.n_tiles = (int64_t)(var.cu_seqlens != nullptr ? 1 : B) * p.n_pairs * H;
  p.var = var;
  const int sms = sm_count_of_current_device();
  const int grid = (int)(p.n_tiles < sms ? p.n_tiles : sms);
  if (is_bf16) {
    ATMA_CUDA_OK(cudaFuncSetAttribute(scan_local_sm100_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes));
    scan_local_sm100_kernel<true><<<grid, kThreads, kSmemBytes, st>>>(mq, mk, mv, p);
  } else {
    ATMA_CUDA_OK(cudaFuncSetAttribute(scan_local_sm100_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes));
    scan_local_sm100_kernel<false><<<grid, kThreads, kSmemBytes, st>>>(mq, mk, mv, p);
  }
  return launch_status("gated_delta_scan (chunk-local, tcgen05)");
}

int scan_local_status_fetch_and_clear(int* out) {
  int v = 0, zero = 0;
  ATMA_CUDA_OK(cudaMemcpyFromSymbol(&v, g_local_status, sizeof(int)));
  if (v != 0) ATMA_CUDA_OK(cudaMemcpyToSymbol(g_local_status, &zero, sizeof(int)));
  *out = v;
  return ATMA_OK;
}

}  // namespace atma
