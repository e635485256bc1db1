// Polar Attention prefill on the 5th-generation tensor cores (sm_100a): tcgen05.mma with TMEM
// accumulators, operands staged by TMA, softmax statistics in registers.
//
// One CTA owns TWO 128-row query tiles that read the same K/V head - two query heads of one
// GQA group over the same rows when the group size is even, else two consecutive row tiles of
// one head - so every K/V tile brought into shared memory feeds two S = Q K^T and two
// O += P V products, and the two tiles ping-pong: while the softmax warps of one tile work on
// their S, the tensor core runs the other tile's products.
//
//   warp 0      TMA producer: Q tiles once, then K and V tiles through 2-stage rings
//   warp 1      MMA issuer (one lane): S_t = Q_t K_j^T (SS), O_t += P_t V_j (P read from TMEM)
//   warps 2-3   idle (they complete the first warpgroup, whose registers are handed over)
//   warps 4-7   softmax + epilogue of tile 0, one thread per query row (= one TMEM lane)
//   warps 8-11  softmax + epilogue of tile 1
// The first warpgroup shrinks to 88 registers per thread (setmaxnreg) so that each softmax
// thread can hold its whole 128-column S row in registers.
//
// TMEM (512 columns): S_0 [0,128) S_1 [128,256) O_0 [256,384) O_1 [384,512); P_t (16-bit,
// two values per column) overwrites the first 64 columns of S_t once the row has been read.
// Per row the kernel streams (m, L = sum p, Q2 = sum p^2, O = sum p v) in the log2 domain with
// the per-row temperature folded into one FMA before ex2; the running maximum used for the
// exponent is only moved when it grew by more than 2^8 (all statistics stay in one frame, so
// the result is unchanged), which keeps the read-modify-write of O out of most iterations.
// Every mbarrier wait is bounded; on expiry the CTA frees its TMEM, returns and leaves a
// status word for the host.
#include "polar_prefill.cuh"
#include "sm100.cuh"
#include "gated_delta_scan.cuh"

namespace atma {

using namespace sm100;

namespace {

constexpr int kBM = 128, kBN = 128, kDK = 128;
constexpr int kStages = 2;
constexpr int kTileBytes = kBM * kDK * 2;             // 32 KiB: two 64-column swizzled boxes
constexpr int kThreads = 384;                        // 3 warpgroups: (TMA, MMA, 2 idle) + 2 x softmax
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;
constexpr float kNegInit = -1.0e30f;                  // "no key seen yet" in the log2 domain
constexpr float kLazyThreshold = 8.0f;

struct Params {
  void* c; int64_t c_sb, c_sh, c_st;
  void* mag; int64_t mag_sb, mag_sh, mag_st;
  const float* n_keys; float n_base; float key_offset;
  const float *v_null, *spg, *null_base, *sps, *beta;
  const float *si_m, *si_l, *si_q2, *si_s;
  float *so_m, *so_l, *so_q2, *so_s;
  int finalize, B, H, Hkv, Tq, Tk, window;
  float eps;
  const int32_t *tile_seq_start, *tile_q_start, *tile_seq_len;
  int n_tiles;
  int pair_heads, n_row_tiles, is_bf16;
  int qpos[3], kpos[3], vpos[3];                     // tensor-map coordinate slot of (t, h, b)
};

__device__ int g_sm100_status = 0;

struct Barriers {
  uint64_t q_full[2];
  uint64_t k_full[kStages], k_empty[kStages], v_full[kStages], v_empty[kStages];
  uint64_t s_full[2], p_full[2], o_final[2];
};

__device__ __forceinline__ void tma_tile(void* dst, const CUtensorMap* m, uint64_t* bar, const int (&pos)[3],
                                         int row, int head, int b) {
  // coordinate slot k (1..3) holds whichever of (row, head, b) the host sorted into it
  const int c1 = pos[0] == 1 ? row : (pos[1] == 1 ? head : b);
  const int c2 = pos[0] == 2 ? row : (pos[1] == 2 ? head : b);
  const int c3 = pos[0] == 3 ? row : (pos[1] == 3 ? head : b);
#pragma unroll
  for (int half = 0; half < 2; ++half)
    tma_load_4d(static_cast<uint8_t*>(dst) + half * (kTileBytes / 2), m, bar, half * 64, c1, c2, c3);
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

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ float max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}

template <bool kBf16>
__global__ void __launch_bounds__(kThreads, 1)
polar_prefill_sm100_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                           const __grid_constant__ CUtensorMap tmap_v, const Params p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;                                  // [2][32K]
  uint8_t* sK = smem + 2 * kTileBytes;                 // [kStages][32K]
  uint8_t* sV = sK + kStages * kTileBytes;             // [kStages][32K]
  __shared__ Barriers bar;
  __shared__ uint32_t s_tmem_base;
  __shared__ int s_abort;
  __shared__ float s_wmin[2][4], s_wmax[2][4];

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const bool packed = p.n_tiles > 0;

  // ---- the two query tiles of this CTA ---------------------------------------------------------
  int row0[2], head[2], q_limit, k_limit, seq_row0 = 0;
  const int b = blockIdx.z;
  if (packed) {
    const int t = blockIdx.x;
    seq_row0 = p.tile_seq_start[t];
    q_limit = p.tile_seq_len[t];
    k_limit = q_limit;
    row0[0] = p.tile_q_start[t];
    if (p.pair_heads) { row0[1] = row0[0]; head[0] = 2 * blockIdx.y; head[1] = head[0] + 1; }
    else { row0[1] = q_limit; head[0] = head[1] = blockIdx.y; }                 // single tile
  } else {
    q_limit = p.Tq; k_limit = p.Tk;
    if (p.pair_heads) {
      row0[0] = row0[1] = (p.n_row_tiles - 1 - (int)blockIdx.x) * kBM;            // long rows first
      head[0] = 2 * blockIdx.y; head[1] = head[0] + 1;
    } else {
      const int pairs = (p.n_row_tiles + 1) / 2;
      const int pr = pairs - 1 - (int)blockIdx.x;
      row0[0] = (2 * pr) * kBM; row0[1] = (2 * pr + 1) * kBM;
      head[0] = head[1] = blockIdx.y;
    }
  }
  const int kvh = head[0] / (p.H / p.Hkv);
  const bool carry_in = p.si_m != nullptr;

  // ---- barriers, TMEM --------------------------------------------------------------------------
  if (tid == 0) {
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bar.q_full[i], 1); mbar_init(&bar.s_full[i], 1);
      mbar_init(&bar.p_full[i], 4); mbar_init(&bar.o_final[i], 1);
    }
    for (int i = 0; i < kStages; ++i) {
      mbar_init(&bar.k_full[i], 1); mbar_init(&bar.k_empty[i], 1);
      mbar_init(&bar.v_full[i], 1); mbar_init(&bar.v_empty[i], 1);
    }
    s_abort = 0;
    fence_barrier_init();
  }
  if (warp == 0) {
    if (lane == 0) { prefetch_tensormap(&tmap_q); prefetch_tensormap(&tmap_k); prefetch_tensormap(&tmap_v); }
    __syncwarp();
    tmem_alloc(&s_tmem_base, 512);
  }

  // ---- per-row scalars (softmax threads) and the key range of each tile ---------------------------
  const int sm_tile = (warp >= 8) ? 1 : 0;             // meaningful for warps >= 4
  const int r_in_tile = 32 * (warp & 3) + lane;        // TMEM lane of this thread
  float n_i = 0.f;
  bool row_ok = false;
  int my_row = 0;
  if (warp >= 4) {
    my_row = (sm_tile ? row0[1] : row0[0]) + r_in_tile;
    row_ok = my_row < q_limit;
    if (row_ok) n_i = packed ? (float)(my_row + 1) : (p.n_keys ? p.n_keys[my_row] : p.n_base + (float)(my_row + 1));
    float mn = row_ok ? n_i : 3.0e38f, mx = row_ok ? n_i : -1.0f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, o));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    }
    if (lane == 0) { s_wmin[sm_tile][warp & 3] = mn; s_wmax[sm_tile][warp & 3] = mx; }
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tbase = s_tmem_base;

  int lo[2], hi[2];
#pragma unroll
  for (int t = 0; t < 2; ++t) {
    float mn = fminf(fminf(s_wmin[t][0], s_wmin[t][1]), fminf(s_wmin[t][2], s_wmin[t][3]));
    float mx = fmaxf(fmaxf(s_wmax[t][0], s_wmax[t][1]), fmaxf(s_wmax[t][2], s_wmax[t][3]));
    int hk = (int)fminf((float)k_limit, ceilf(mx - p.key_offset));
    hk = max(hk, 0);
    hi[t] = (hk + kBN - 1) / kBN;
    lo[t] = 0;
    if (p.window > 0) {
      const float first = mn - (float)p.window - p.key_offset;
      if (first > 0.f) lo[t] = (int)first / kBN;
    }
    if (row0[t] >= q_limit) hi[t] = 0;
    if (lo[t] > hi[t]) lo[t] = hi[t];
  }
  int jmin, jmax;
  {
    const bool a0 = hi[0] > lo[0], a1 = hi[1] > lo[1];
    jmin = a0 ? (a1 ? min(lo[0], lo[1]) : lo[0]) : (a1 ? lo[1] : 0);
    jmax = a0 ? (a1 ? max(hi[0], hi[1]) : hi[0]) : (a1 ? hi[1] : 0);
  }
  // all per-tile scalars are selected with ternaries so that they stay in registers
  auto active = [&](int t, int j) { return t ? (j >= lo[1] && j < hi[1]) : (j >= lo[0] && j < hi[0]); };
  volatile int* abort_flag = &s_abort;

  if (warp < 4) {
  // Register hand-over: 88 x 128 + 208 x 256 = 168 x 384, the pool this CTA is launched with (ptxas -v: 168 registers
  // under __launch_bounds__(384, 1)).  The sum must not exceed that pool, or the last setmaxnreg.inc never returns.
  asm volatile("setmaxnreg.dec.sync.aligned.u32 88;");
  if (warp == 0) {
    // =============================== TMA producer ================================================
    if (lane == 0) {
#pragma unroll
      for (int t = 0; t < 2; ++t) {
        if (hi[t] > lo[t]) {
          mbar_arrive_expect_tx(&bar.q_full[t], kTileBytes);
          tma_tile(sQ + t * kTileBytes, &tmap_q, &bar.q_full[t], p.qpos, seq_row0 + row0[t], head[t], b);
        }
      }
      for (int j = jmin; j < jmax; ++j) {
        const int it = j - jmin, s = it % kStages;
        const uint32_t ph = (uint32_t)(it / kStages) & 1u;
        if (!mbar_wait(&bar.k_empty[s], ph ^ 1u, abort_flag)) break;
        mbar_arrive_expect_tx(&bar.k_full[s], kTileBytes);
        tma_tile(sK + s * kTileBytes, &tmap_k, &bar.k_full[s], p.kpos, seq_row0 + j * kBN, kvh, b);
        if (!mbar_wait(&bar.v_empty[s], ph ^ 1u, abort_flag)) break;
        mbar_arrive_expect_tx(&bar.v_full[s], kTileBytes);
        tma_tile(sV + s * kTileBytes, &tmap_v, &bar.v_full[s], p.vpos, seq_row0 + j * kBN, kvh, b);
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // =============================== MMA issuer =================================================
    if (lane == 0) {
      constexpr uint32_t idesc_qk = make_idesc(kBM, kBN, kBf16 ? 1 : 0, 0, 0);
      constexpr uint32_t idesc_pv = make_idesc(kBM, kDK, kBf16 ? 1 : 0, 0, 1);
      const uint32_t q_addr = smem_u32(sQ), k_addr = smem_u32(sK), v_addr = smem_u32(sV);
      bool ok = true;
      // One thread issues all MMAs, so the issue sequence has to be short: the loops are unrolled
      // and each descriptor is its tile's base descriptor plus a compile-time constant (the
      // 14-bit address field cannot carry out: shared memory addresses stay below 256 KiB).
      const uint64_t desc_hi_k = (uint64_t(1024 >> 4) << 32) | (uint64_t(1) << 46) | (uint64_t(2) << 61) | (uint64_t(16 >> 4) << 16);
      const uint64_t desc_hi_v = (uint64_t(1024 >> 4) << 32) | (uint64_t(1) << 46) | (uint64_t(2) << 61) |
                                 (uint64_t((kTileBytes / 2) >> 4) << 16);
      auto issue_qk = [&](int t, int s) {
        const uint64_t a0 = desc_hi_k | uint64_t(((q_addr + t * kTileBytes) >> 4) & 0x3FFFu);
        const uint64_t b0 = desc_hi_k | uint64_t(((k_addr + s * kTileBytes) >> 4) & 0x3FFFu);
#pragma unroll
        for (int kk = 0; kk < kDK / 16; ++kk) {
          constexpr int dummy = 0; (void)dummy;
          const uint64_t off = uint64_t(((kk >> 2) * (kTileBytes / 2) + (kk & 3) * 32) >> 4);   // compile-time constant
          mma_ss(tbase + t * 128, a0 + off, b0 + off, idesc_qk, kk > 0);
        }
      };
      auto issue_pv = [&](int t, int s, bool acc) {
        const uint64_t b0 = desc_hi_v | uint64_t(((v_addr + s * kTileBytes) >> 4) & 0x3FFFu);
        const uint32_t pa = tbase + t * 128, od = tbase + 256 + t * 128;
#pragma unroll
        for (int kk = 0; kk < kBN / 16; ++kk)
          mma_ts(od, pa + kk * 8, b0 + uint64_t(kk * (2048 >> 4)), idesc_pv, (kk > 0 || acc) ? 1u : 0u);
      };
      if (jmax > jmin) {
#pragma unroll
        for (int t = 0; t < 2; ++t)
          if (ok && hi[t] > lo[t]) ok = mbar_wait(&bar.q_full[t], 0, abort_flag);
        // prologue: S for the first key tile
        if (ok) ok = mbar_wait(&bar.k_full[0], 0, abort_flag);
        if (ok) {
          tc_fence_after();
#pragma unroll
          for (int t = 0; t < 2; ++t)
            if (active(t, jmin)) { issue_qk(t, 0); tc_commit(&bar.s_full[t]); }
          tc_commit(&bar.k_empty[0]);
        }
        for (int j = jmin; j < jmax && ok; ++j) {
          const int it = j - jmin, s = it % kStages, s1 = (it + 1) % kStages;
          const uint32_t ph = (uint32_t)(it / kStages) & 1u, ph1 = (uint32_t)((it + 1) / kStages) & 1u;
          bool v_ready = false, k1_ready = false;
#pragma unroll
          for (int t = 0; t < 2; ++t) {
            if (ok && active(t, j)) {
              ok = mbar_wait(&bar.p_full[t], (uint32_t)(j - lo[t]) & 1u, abort_flag);
              if (ok && !v_ready) { ok = mbar_wait(&bar.v_full[s], ph, abort_flag); v_ready = true; }
              if (ok) {
                tc_fence_after();
                issue_pv(t, s, carry_in || j > lo[t]);
                if (!active(t, j + 1)) tc_commit(&bar.o_final[t]);
              }
            }
            if (ok && active(t, j + 1)) {
              if (!k1_ready) { ok = mbar_wait(&bar.k_full[s1], ph1, abort_flag); k1_ready = true; }
              if (ok) {
                tc_fence_after();
                issue_qk(t, s1);
                tc_commit(&bar.s_full[t]);
              }
            }
          }
          // keep the stage barriers in step even when no tile used this stage
          if (ok && !v_ready) ok = mbar_wait(&bar.v_full[s], ph, abort_flag);
          if (ok && !k1_ready && j + 1 < jmax) ok = mbar_wait(&bar.k_full[s1], ph1, abort_flag);
          if (!ok) break;
          tc_commit(&bar.v_empty[s]);
          if (j + 1 < jmax) tc_commit(&bar.k_empty[s1]);
        }
      }
    }
    __syncwarp();
  }
  } else {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 208;");
    // =============================== softmax + epilogue ===========================================
    const int t = sm_tile;
    const int h = t ? head[1] : head[0];
    const int my_lo = t ? lo[1] : lo[0], my_hi = t ? hi[1] : hi[0], my_row0 = t ? row0[1] : row0[0];
    const uint32_t lane_base = tbase + (uint32_t(32 * (warp & 3)) << 16);
    const uint32_t tS = lane_base + t * 128, tO = lane_base + 256 + t * 128;
    const float n_clamped = fmaxf(p.window > 0 ? fminf(n_i, (float)p.window) : n_i, 1.0f);
    const float temp = 1.0f + p.spg[h] * logf(n_clamped);
    const float sc2 = temp * rsqrtf((float)kDK) * kLog2e;
    const int n_iter = my_hi - my_lo;
    const int64_t srow = ((int64_t)b * p.H + h) * p.Tq + my_row;     // dense statistics index

    float m_used = kNegInit, m_run = kNegInit, L = 0.f, Q2 = 0.f;
    bool ok = true;
    bool o_live = false;                                            // O_t holds data (warp-uniform)
    if (carry_in && my_row0 < q_limit) {
      if (row_ok) {
        const float mi = p.si_m[srow];
        m_used = m_run = (mi <= -1.0e37f) ? kNegInit : mi * kLog2e;
        L = p.si_l[srow]; Q2 = p.si_q2[srow];
      }
#pragma unroll 1
      for (int ch = 0; ch < 4; ++ch) {
        uint32_t r[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) r[i] = row_ok ? __float_as_uint(p.si_s[srow * kDK + ch * 32 + i]) : 0u;
        tmem_st32(tO + ch * 32, r);
      }
      tmem_st_wait();
      o_live = true;
    }

    for (int j = my_lo; j < my_hi; ++j) {
      ok = mbar_wait(&bar.s_full[t], (uint32_t)(j - my_lo) & 1u, abort_flag);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      // key column c of this tile is visible iff c_lo <= c < c_hi
      const float kbase = (float)(j * kBN) + p.key_offset;
      const float c_hi = fminf(n_i - kbase, (float)(k_limit - j * kBN));
      const float c_lo = p.window > 0 ? (n_i - (float)p.window - kbase) : -1.0f;
      const bool full = row_ok && c_hi >= (float)kBN && c_lo <= 0.0f;
      const float c_hi_eff = row_ok ? c_hi : 0.0f;

      // the whole S row in registers: four loads in flight, one wait
      uint32_t r[kBN];
#pragma unroll
      for (int ch = 0; ch < 4; ++ch) tmem_ld32_nowait(tS + ch * 32, &r[ch * 32]);
      tmem_ld_wait();
#pragma unroll
      for (int i = 0; i < kBN; ++i) reg_fence(r[i]);
      if (!full) {                                                  // diagonal / window-edge / ragged tile
#pragma unroll
        for (int i = 0; i < kBN; ++i) {
          const float cc = (float)i;
          if (!(cc >= c_lo && cc < c_hi_eff)) r[i] = 0xff800000u;   // -inf
        }
      }
      float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
#pragma unroll
      for (int i = 0; i < kBN; i += 8) {
        mx0 = max3(mx0, __uint_as_float(r[i]), __uint_as_float(r[i + 1]));
        mx1 = max3(mx1, __uint_as_float(r[i + 2]), __uint_as_float(r[i + 3]));
        mx2 = max3(mx2, __uint_as_float(r[i + 4]), __uint_as_float(r[i + 5]));
        mx3 = max3(mx3, __uint_as_float(r[i + 6]), __uint_as_float(r[i + 7]));
      }
      const float m_cand = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3)) * sc2;   // -inf if nothing visible
      const float m_new = fmaxf(m_run, m_cand);
      m_run = m_new;
      if (__any_sync(0xffffffffu, (m_new - m_used) > kLazyThreshold)) {
        const float alpha = ex2(m_used - m_new);
        L *= alpha; Q2 *= alpha * alpha;
        if (o_live) {
#pragma unroll 1
          for (int ch = 0; ch < 4; ++ch) {
            uint32_t o[32];
            tmem_ld32(tO + ch * 32, o);
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
            tmem_st32(tO + ch * 32, o);
          }
        }
        m_used = m_new;
      }
      // p = 2^(s*sc2 - m_used), statistics, P tile (16-bit) over the first 64 S columns
      const float neg_m = -m_used;
      // Two columns per instruction with the packed fp32x2 FMA/ADD of sm_100: per pair of
      // elements one FFMA2 (exponent argument), two ex2, one FADD2 (L), one FFMA2 (Q2), one pack.
      const float2 sc2v = make_float2(sc2, sc2), negv = make_float2(neg_m, neg_m);
      float2 la = make_float2(0.f, 0.f), lb = la, qa = la, qb = la;
#pragma unroll
      for (int ch = 0; ch < 4; ++ch) {
        uint32_t pk[16];
#pragma unroll
        for (int i = 0; i < 32; i += 4) {
          const float2 x0 = __ffma2_rn(make_float2(__uint_as_float(r[ch * 32 + i]), __uint_as_float(r[ch * 32 + i + 1])), sc2v, negv);
          const float2 x1 = __ffma2_rn(make_float2(__uint_as_float(r[ch * 32 + i + 2]), __uint_as_float(r[ch * 32 + i + 3])), sc2v, negv);
          const float2 p0 = make_float2(ex2(x0.x), ex2(x0.y));
          const float2 p1 = make_float2(ex2(x1.x), ex2(x1.y));
          la = __fadd2_rn(la, p0); lb = __fadd2_rn(lb, p1);
          qa = __ffma2_rn(p0, p0, qa); qb = __ffma2_rn(p1, p1, qb);
          pk[i >> 1] = pack2<kBf16>(p0.x, p0.y);
          pk[(i >> 1) + 1] = pack2<kBf16>(p1.x, p1.y);
        }
        tmem_st16(tS + ch * 16, pk);
      }
      const float l0 = la.x + la.y, l1 = lb.x + lb.y, q0 = qa.x + qa.y, q1 = qb.x + qb.y;
      L += l0 + l1; Q2 += q0 + q1;
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();                                                 // one arrival per warp, not per thread
      if (lane == 0) mbar_arrive(&bar.p_full[t]);
      o_live = true;
    }

    // ---- epilogue -------------------------------------------------------------------------------
    if (ok && n_iter > 0) {
      ok = mbar_wait(&bar.o_final[t], 0, abort_flag);
      ok = __all_sync(0xffffffffu, ok);
      tc_fence_after();
    }
    if (ok && my_row0 < q_limit) {
      const bool have_o = o_live;                                   // else O is all zero
      if (!p.finalize) {
        if (row_ok) {
          p.so_m[srow] = (m_used <= kNegInit) ? -1.0e38f : m_used * kLn2;
          p.so_l[srow] = L; p.so_q2[srow] = Q2;
        }
#pragma unroll 1
        for (int ch = 0; ch < 4; ++ch) {
          uint32_t r[32];
          if (have_o) tmem_ld32(tO + ch * 32, r);
          if (row_ok) {
#pragma unroll
            for (int i = 0; i < 32; i += 4) {
              float4 v = have_o ? make_float4(__uint_as_float(r[i]), __uint_as_float(r[i + 1]),
                                              __uint_as_float(r[i + 2]), __uint_as_float(r[i + 3]))
                                : make_float4(0.f, 0.f, 0.f, 0.f);
              *reinterpret_cast<float4*>(p.so_s + srow * kDK + ch * 32 + i) = v;
            }
          }
        }
      } else {
        const float a_n = temp * (p.null_base[h] + p.sps[h] * sqrtf(logf(n_clamped + 1.0f))) * kLog2e;
        const float m_fin = fmaxf(m_used, a_n);
        const float alpha = ex2(m_used - m_fin);
        const float Lf = L * alpha, Q2f = Q2 * alpha * alpha;
        const float p_n = ex2(a_n - m_fin);
        const float Z = Lf + p_n;
        const float* vn = p.v_null + h * kDK;
        float sq = 0.f;
#pragma unroll 1
        for (int ch = 0; ch < 4; ++ch) {
          uint32_t r[32];
          if (have_o) tmem_ld32(tO + ch * 32, r);
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const float s = (have_o ? __uint_as_float(r[i]) * alpha : 0.f) + p_n * vn[ch * 32 + i];
            sq = fmaf(s, s, sq);
          }
        }
        const float inv = 1.0f / fmaxf(sqrtf(sq), p.eps);
        uint16_t* crow = reinterpret_cast<uint16_t*>(p.c) + b * p.c_sb + h * p.c_sh + (int64_t)(seq_row0 + my_row) * p.c_st;
#pragma unroll 1
        for (int ch = 0; ch < 4; ++ch) {
          uint32_t r[32];
          if (have_o) tmem_ld32(tO + ch * 32, r);
          uint32_t o16[16];
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            const float s0 = (have_o ? __uint_as_float(r[i]) * alpha : 0.f) + p_n * vn[ch * 32 + i];
            const float s1 = (have_o ? __uint_as_float(r[i + 1]) * alpha : 0.f) + p_n * vn[ch * 32 + i + 1];
            o16[i >> 1] = pack2<kBf16>(s0 * inv, s1 * inv);
          }
          if (row_ok) {
#pragma unroll
            for (int i = 0; i < 16; i += 4)
              *reinterpret_cast<uint4*>(crow + ch * 32 + i * 2) = make_uint4(o16[i], o16[i + 1], o16[i + 2], o16[i + 3]);
          }
        }
        if (row_ok) {
          const float n_eff = Lf * Lf / fmaxf(Q2f, 1e-30f);
          const float m_eff = n_eff * (Lf / fmaxf(Z, p.eps));
          const float mg = tanhf(p.beta[h] * log1pf(m_eff));
          uint16_t* mp = reinterpret_cast<uint16_t*>(p.mag) + b * p.mag_sb + h * p.mag_sh + (int64_t)(seq_row0 + my_row) * p.mag_st;
          *mp = (uint16_t)(pack2<kBf16>(mg, 0.f) & 0xffffu);
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (tid == 0 && s_abort) atomicExch(&g_sm100_status, 1);
  if (warp == 0) tmem_dealloc(tbase, 512);
}

// Sort the three outer dimensions (t, h, b) by stride so that the tensor map has increasing
// strides whatever the storage order; `pos` receives the coordinate slot of each.
int build_map(CUtensorMap* out, const void* base, int is_bf16, int64_t T, int64_t Hn, int64_t Bn, int64_t st,
              int64_t sh, int64_t sb, int pos[3]) {
  struct D { int64_t size, stride; int which; };
  D d[3] = {{T, st, 0}, {Hn, sh, 1}, {Bn, sb, 2}};
  // a dimension of extent 1 has no meaningful stride: give it a dense one so that it sorts last
  int64_t span = kDK;
  for (int i = 0; i < 3; ++i) if (d[i].size > 1) span = std::max<int64_t>(span, d[i].size * d[i].stride);
  for (int i = 0; i < 3; ++i) if (d[i].size <= 1) { d[i].size = 1; d[i].stride = span; }
  for (int i = 0; i < 3; ++i)
    for (int j = i + 1; j < 3; ++j)
      if (d[j].stride < d[i].stride) { D tmp = d[i]; d[i] = d[j]; d[j] = tmp; }
  uint64_t dims[4] = {(uint64_t)kDK, (uint64_t)d[0].size, (uint64_t)d[1].size, (uint64_t)d[2].size};
  int64_t strides[3] = {d[0].stride, d[1].stride, d[2].stride};
  uint32_t box[4] = {64, 1, 1, 1};
  for (int i = 0; i < 3; ++i) {
    pos[d[i].which] = i + 1;
    if (d[i].which == 0) box[i + 1] = kBM;
  }
  return make_tmap_16bit_4d(out, base, is_bf16, dims, strides, box);
}

bool aligned16(const void* ptr, int64_t a, int64_t b2, int64_t c) {
  return (reinterpret_cast<uintptr_t>(ptr) % 16 == 0) && a % 8 == 0 && b2 % 8 == 0 && c % 8 == 0;
}

}  // namespace

bool polar_prefill_sm100_supported(const atma_polar_prefill_args& a) {
  if (!(a.dtype == ATMA_BF16 || a.dtype == ATMA_F16) || a.dk != kDK) return false;
  if (a.q == nullptr) return true;                       // shape-only query
  if (!aligned16(a.q, a.q_st, a.q_sh, a.B > 1 ? a.q_sb : 0)) return false;
  if (!aligned16(a.k, a.k_st, a.k_sh, a.B > 1 ? a.k_sb : 0)) return false;
  if (!aligned16(a.v, a.v_st, a.v_sh, a.B > 1 ? a.v_sb : 0)) return false;
  if (a.finalize && (reinterpret_cast<uintptr_t>(a.c) % 16 != 0 || a.c_st % 8 != 0 || a.c_sh % 8 != 0 || a.c_sb % 8 != 0))
    return false;
  return true;
}

int polar_prefill_sm100(const atma_polar_prefill_args& a, cudaStream_t st) {
  Params p{};
  p.c = a.c; p.c_sb = a.c_sb; p.c_sh = a.c_sh; p.c_st = a.c_st;
  p.mag = a.mag; p.mag_sb = a.mag_sb; p.mag_sh = a.mag_sh; p.mag_st = a.mag_st;
  p.n_keys = a.n_keys; p.n_base = a.n_base; p.key_offset = (float)a.key_offset;
  p.v_null = a.v_null; p.spg = a.spg; p.null_base = a.null_base; p.sps = a.sps; p.beta = a.beta;
  p.si_m = a.stats_in_m; p.si_l = a.stats_in_l; p.si_q2 = a.stats_in_q2; p.si_s = a.stats_in_s;
  p.so_m = a.stats_out_m; p.so_l = a.stats_out_l; p.so_q2 = a.stats_out_q2; p.so_s = a.stats_out_s;
  p.finalize = a.finalize; p.B = a.B; p.H = a.H; p.Hkv = a.Hkv; p.Tq = a.Tq; p.Tk = a.Tk;
  p.window = a.window; p.eps = a.eps;
  p.tile_seq_start = a.tile_seq_start; p.tile_q_start = a.tile_q_start; p.tile_seq_len = a.tile_seq_len;
  p.n_tiles = a.n_tiles;
  p.is_bf16 = a.dtype == ATMA_BF16;
  const int G = a.H / a.Hkv;
  p.pair_heads = (G % 2 == 0) ? 1 : 0;
  p.n_row_tiles = (a.Tq + kBM - 1) / kBM;

  CUtensorMap mq, mk, mv;
  int rc = build_map(&mq, a.q, p.is_bf16, a.Tq, a.H, a.B, a.q_st, a.q_sh, a.q_sb, p.qpos);
  if (rc == ATMA_OK) rc = build_map(&mk, a.k, p.is_bf16, a.Tk, a.Hkv, a.B, a.k_st, a.k_sh, a.k_sb, p.kpos);
  if (rc == ATMA_OK) rc = build_map(&mv, a.v, p.is_bf16, a.Tk, a.Hkv, a.B, a.v_st, a.v_sh, a.v_sb, p.vpos);
  if (rc != ATMA_OK) return rc;

  dim3 grid;
  if (a.n_tiles > 0) grid = dim3(a.n_tiles, p.pair_heads ? a.H / 2 : a.H, 1);
  else if (p.pair_heads) grid = dim3(p.n_row_tiles, a.H / 2, a.B);
  else grid = dim3((p.n_row_tiles + 1) / 2, a.H, a.B);
  const int smem = (2 + 2 * kStages) * kTileBytes + 1024;
  if (p.is_bf16) {
    ATMA_CUDA_OK(cudaFuncSetAttribute(polar_prefill_sm100_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    polar_prefill_sm100_kernel<true><<<grid, kThreads, smem, st>>>(mq, mk, mv, p);
  } else {
    ATMA_CUDA_OK(cudaFuncSetAttribute(polar_prefill_sm100_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    polar_prefill_sm100_kernel<false><<<grid, kThreads, smem, st>>>(mq, mk, mv, p);
  }
  return launch_status("polar_prefill (tcgen05 kernel)");
}

int sm100_status_fetch_and_clear(int* out) {
  int v = 0, zero = 0;
  ATMA_CUDA_OK(cudaMemcpyFromSymbol(&v, g_sm100_status, sizeof(int)));
  if (v != 0) ATMA_CUDA_OK(cudaMemcpyToSymbol(g_sm100_status, &zero, sizeof(int)));
  *out = v;
  return ATMA_OK;
}

}  // namespace atma


// Non-zero if a tensor-core kernel gave up on a bounded wait since the last call (synchronises
// the device; clears the flag).
extern "C" int atma_device_status(int* status) {
  ATMA_REQUIRE(status != nullptr, "device_status: null out pointer");
  int a = 0, b = 0, c = 0;
  int rc = atma::sm100_status_fetch_and_clear(&a);
  if (rc == ATMA_OK) rc = atma::scan_sm100_status_fetch_and_clear(&b);
  if (rc == ATMA_OK) rc = atma::scan_local_status_fetch_and_clear(&c);
  *status = a | b | c;
  return rc;
}
