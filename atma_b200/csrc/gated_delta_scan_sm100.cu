// Gated-delta scan, the recurrence over chunks, on the 5th-generation tensor cores (sm_100a):
// tcgen05.mma with TMEM accumulators, per-chunk factor records brought in by TMA.
//
// One CTA owns one (recurrence, head) and the whole state S [dk][dv], held TRANSPOSED: every
// thread of the eight state warps keeps 64 fp32 values of one row of S^T [v][k] in registers for
// the whole sequence.  Per 64-token chunk, with the state-independent factors -W, Qg, Kt, U0^T, Rq
// of gated_delta_scan.cuh (s, p = rows of the chunk; k, v = key / value channel):
//
//   MMA1a  U^T  = S^T (-W)^T            M=128 (v) N=64 (s)  K=128 (k)
//   MMA1b  O^T  = S^T Qg^T              M=128 (v) N=64 (p)  K=128 (k)
//   threads     U^T += U0^T -> 16-bit, back into TMEM
//   MMA2a  dS^T = U^T Kt                M=128 (v) N=128 (k) K=64 (s);  threads: S^T = g_C S^T + dS^T
//   MMA2b  O^T += U^T Rq^T              M=128 (v) N=64 (p)  K=64 (s)
//
// The A operand of every product (the 16-bit copies of S^T and U^T) is read from TMEM, where the
// state warps put it with tcgen05.st; only the B operands (the record tiles, exactly as TMA
// delivers them) come from shared memory.  One SM's shared-memory bandwidth is what bounds this
// kernel, so nothing the threads produce goes through shared memory, and no thread-written tile
// needs a proxy fence.  All four accumulators have the value channel v on the 128 TMEM lanes, which
// spreads both thread phases of the chunk-to-chunk critical path over all four warp schedulers.
//
//   warp 0      TMA producer: the pieces of each chunk record through a 3-stage ring
//   warp 1      MMA issuer (one lane); owns the TMEM allocation
//   warps 2-9   state warps; warp w works on TMEM lanes 32 (w % 4) .. +31 and on column half
//               (w - 2) / 4 of whatever it reads (k for S^T, s for U^T, p for O^T)
// TMEM (512 columns allocated): 16-bit S^T [0,64) | 16-bit U^T [64,96) | U^T fp32 [128,192) |
// O^T_0 [192,256) | O^T_1 [256,320) | dS^T [320,448).
// Every mbarrier wait is bounded; on expiry the CTA frees its TMEM, returns and leaves a status
// word for the host.
#include "common.cuh"
#include "sm100.cuh"
#include "gated_delta_scan.cuh"

namespace atma {

using namespace sm100;
using namespace scan;

namespace {

__device__ int g_scan_status = 0;

constexpr int kThreads = 320;
constexpr int kA1Bytes = 2 * kD * 128;            // [-W ; Qg]: [128 rows][128 k] 16-bit = two 64-column boxes of 16 KiB
constexpr int kKtBytes = 2 * kC * 128;            // [64 s][128 k] = two boxes of 8 KiB
constexpr int kU0Bytes = kD * 128;                // U0^T: [128 v][64 s], one box
constexpr int kRqBytes = kC * 128;                // [64 p][64 s], one box
constexpr int kStageBytes = kA1Bytes + kKtBytes + kU0Bytes + kRqBytes;   // 72 KiB
constexpr int kStages = 3;
constexpr int kSmemBytes = kStages * kStageBytes + 1024;
constexpr int kRecRows = kRecBytes / 256;         // a record as rows of 128 16-bit values (288)
constexpr int kRecRowsRq = kRecBytes / 128;       // ... and as rows of 64 values (576)
constexpr uint32_t kColSb = 0, kColUb = 64, kColU = 128, kColO = 192, kColS = 320;

struct Barriers {
  uint64_t a1_full[kStages], a1_empty[kStages], y_full[kStages], y_empty[kStages];
  uint64_t o_free[2], o_done[2];
  uint64_t sb_ready, ub_ready, u_full, s_done;
};

struct Params {
  const float* gcs;
  const float* initial_state;
  void* o;
  float* final_state;
  int Tlen, H, NC, is_bf16;
  RecMap map;
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

// byte offset of the 16-byte chunk `chunk` (0..7) of row `row` inside a 128-byte-swizzled box
__device__ __forceinline__ uint32_t box_off(int row, int chunk) {
  return (uint32_t)(row * 128 + ((chunk ^ (row & 7)) << 4));
}

template <bool kBf16>
__global__ void __launch_bounds__(kThreads, 1)
scan_recur_sm100_kernel(const __grid_constant__ CUtensorMap tmap_rec, const __grid_constant__ CUtensorMap tmap_rq, const Params p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  __shared__ Barriers bar;
  __shared__ uint32_t s_tmem_base;
  __shared__ int s_abort;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int h = blockIdx.x, b = blockIdx.y;
  const bool packed = p.var.cu_seqlens != nullptr;
  const int rb = packed ? 0 : p.map.rec[b];
  const bool zero_u0 = packed ? false : p.map.zero_u0[b] != 0;
  int c_begin, c_end;
  int64_t tok_base, tok_end;
  if (packed) {
    c_begin = p.var.cu_chunks[b]; c_end = p.var.cu_chunks[b + 1];
    tok_base = p.var.cu_seqlens[b]; tok_end = p.var.cu_seqlens[b + 1];
  } else {
    c_begin = p.map.c_begin[b]; c_end = p.map.c_end[b] > 0 ? p.map.c_end[b] : p.NC;
    const int64_t orow0 = (int64_t)max(p.map.o_row[b], 0) * p.Tlen;  // the batch row of o this recurrence writes
    tok_base = orow0 + (int64_t)c_begin * kC;
    tok_end = orow0 + min((int64_t)p.Tlen, (int64_t)c_end * kC);
  }
  const int n_chunks = max(c_end - c_begin, 0);
  const int64_t rec0 = ((int64_t)rb * p.H + h) * p.NC + c_begin;     // first record of this recurrence
  const float* gcs = p.gcs + rec0;
  const bool want_o = p.o != nullptr && (packed || p.map.o_row[b] >= 0);   // a negative row: this recurrence only carries state

  if (tid == 0) {
    for (int i = 0; i < kStages; ++i) {
      mbar_init(&bar.a1_full[i], 1); mbar_init(&bar.a1_empty[i], 1);
      mbar_init(&bar.y_full[i], 1); mbar_init(&bar.y_empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) { mbar_init(&bar.o_free[i], 8); mbar_init(&bar.o_done[i], 1); }
    mbar_init(&bar.sb_ready, 8); mbar_init(&bar.ub_ready, 8);
    mbar_init(&bar.u_full, 1); mbar_init(&bar.s_done, 1);
    s_abort = 0;
    fence_barrier_init();
  }
  if (warp == 1) tmem_alloc(&s_tmem_base, 512);
  if (warp == 0 && lane == 0) { prefetch_tensormap(&tmap_rec); prefetch_tensormap(&tmap_rq); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tbase = s_tmem_base;
  volatile int* abort_flag = &s_abort;

  if (warp == 0) {
    // =============================== TMA producer ================================================
    if (lane == 0) {
      for (int i = 0; i < n_chunks; ++i) {
        const int s = i % kStages;
        const uint32_t ph = (uint32_t)(i / kStages) & 1u;
        uint8_t* st = smem + s * kStageBytes;
        const int row = (int)((rec0 + i) * kRecRows), row64 = (int)((rec0 + i) * kRecRowsRq);
        if (!mbar_wait(&bar.a1_empty[s], ph ^ 1u, abort_flag)) break;
        mbar_arrive_expect_tx(&bar.a1_full[s], kA1Bytes);
#pragma unroll
        for (int half = 0; half < 2; ++half) {                      // -W rows then Qg rows, two column boxes each
          tma_load_4d(st + half * 16384, &tmap_rec, &bar.a1_full[s], half * 64, row, 0, 0);
          tma_load_4d(st + half * 16384 + 8192, &tmap_rec, &bar.a1_full[s], half * 64, row + 64, 0, 0);
        }
        if (!mbar_wait(&bar.y_empty[s], ph ^ 1u, abort_flag)) break;
        mbar_arrive_expect_tx(&bar.y_full[s], kKtBytes + kU0Bytes + kRqBytes);
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          tma_load_4d(st + kA1Bytes + half * 8192, &tmap_rec, &bar.y_full[s], half * 64, row + 128, 0, 0);
          tma_load_4d(st + kA1Bytes + kKtBytes + half * 8192, &tmap_rq, &bar.y_full[s], 0, row64 + 384 + half * 64, 0, 0);
        }
        tma_load_4d(st + kA1Bytes + kKtBytes + kU0Bytes, &tmap_rq, &bar.y_full[s], 0, row64 + 512, 0, 0);
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // =============================== MMA issuer =================================================
    if (lane == 0) {
      constexpr int fmt = kBf16 ? 1 : 0;
      constexpr uint32_t idesc_n64 = make_idesc(128, 64, fmt, 0, 0);     // B = W, Qg or Rq rows, K-major
      constexpr uint32_t idesc_s = make_idesc(128, 128, fmt, 0, 1);      // dS^T = U^T Kt: B = Kt [s][k] MN-major
      const uint64_t hi_k = (uint64_t(1024 >> 4) << 32) | (uint64_t(1) << 46) | (uint64_t(2) << 61) | (uint64_t(16 >> 4) << 16);
      const uint64_t hi_mn64 = (uint64_t(1024 >> 4) << 32) | (uint64_t(1) << 46) | (uint64_t(2) << 61) | (uint64_t(8192 >> 4) << 16);
      bool ok = true;
      for (int i = 0; i < n_chunks && ok; ++i) {
        const int s = i % kStages, ob = i & 1;
        const uint32_t ph = (uint32_t)(i / kStages) & 1u;
        const uint32_t st = smem_u32(smem + s * kStageBytes);
        const uint32_t tO = tbase + kColO + ob * 64;
        const uint64_t a1 = hi_k | uint64_t((st >> 4) & 0x3FFFu);
        ok = mbar_wait(&bar.sb_ready, (uint32_t)i & 1u, abort_flag);
        if (ok) ok = mbar_wait(&bar.a1_full[s], ph, abort_flag);
        if (!ok) break;
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          const uint64_t off = uint64_t(((kk >> 2) * 16384 + (kk & 3) * 32) >> 4);
          mma_ts(tbase + kColU, tbase + kColSb + kk * 8, a1 + off, idesc_n64, kk > 0);
        }
        tc_commit(&bar.u_full);
        if (want_o) {
          if (i >= 2) ok = mbar_wait(&bar.o_free[ob], (uint32_t)((i >> 1) - 1) & 1u, abort_flag);
          if (!ok) break;
          tc_fence_after();
#pragma unroll
          for (int kk = 0; kk < 8; ++kk) {
            const uint64_t off = uint64_t(((kk >> 2) * 16384 + (kk & 3) * 32) >> 4);
            mma_ts(tO, tbase + kColSb + kk * 8, a1 + uint64_t(8192 >> 4) + off, idesc_n64, kk > 0);
          }
        }
        if (i + kStages < n_chunks) tc_commit(&bar.a1_empty[s]);    // nobody waits for the last ones
        ok = mbar_wait(&bar.ub_ready, (uint32_t)i & 1u, abort_flag);
        if (ok) ok = mbar_wait(&bar.y_full[s], ph, abort_flag);
        if (!ok) break;
        tc_fence_after();
        {
          const uint64_t kt0 = hi_mn64 | uint64_t(((st + kA1Bytes) >> 4) & 0x3FFFu);
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)
            mma_ts(tbase + kColS, tbase + kColUb + kk * 8, kt0 + uint64_t((kk * 2048) >> 4), idesc_s, kk > 0);
        }
        tc_commit(&bar.s_done);
        if (want_o) {
          const uint64_t rq0 = hi_k | uint64_t(((st + kA1Bytes + kKtBytes + kU0Bytes) >> 4) & 0x3FFFu);
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)
            mma_ts(tO, tbase + kColUb + kk * 8, rq0 + uint64_t((kk * 32) >> 4), idesc_n64, 1u);
          tc_commit(&bar.o_done[ob]);
        }
        if (i + kStages < n_chunks) tc_commit(&bar.y_empty[s]);
      }
    }
    __syncwarp();
  } else {
    // =============================== state warps ==================================================
    const int quad = warp & 3, half = (warp - 2) >> 2;
    const int row = 32 * quad + lane;                    // TMEM lane = value channel v
    const uint32_t lane_base = tbase + (uint32_t(32 * quad) << 16);

    // where the state comes from and goes to: element (k, v) of the [dk][dv] plane, k = 64*half + j
    const int srow = packed ? b : p.map.state_row[b];
    const int64_t sbase = ((int64_t)srow * p.H + h) * kD * kD + (int64_t)(64 * half) * kD + row;
    const float* s_in = p.initial_state ? p.initial_state + sbase : nullptr;
    float* s_out = p.final_state ? p.final_state + sbase : nullptr;
    if (packed && p.var.state_table != nullptr) {
      float* trow = p.var.state_table + p.var.slots[b] * p.var.slot_stride + (int64_t)h * kD * kD + (int64_t)(64 * half) * kD + row;
      s_in = (p.var.has_initial == nullptr || p.var.has_initial[b] != 0) ? trow : nullptr;
      s_out = trow;
    }
    float* snap_base = nullptr;
    if (packed && p.var.snapshots != nullptr)
      snap_base = p.var.snapshots + ((int64_t)p.var.snap_offsets[b] * p.H + h) * kD * kD + (int64_t)(64 * half) * kD + row;

    float S[64];                                          // S^T[v = row][k = 64*half + j], fp32 master
#pragma unroll
    for (int j = 0; j < 64; ++j) S[j] = s_in ? s_in[(int64_t)j * kD] : 0.f;
    if (n_chunks == 0 && s_out != nullptr && s_out != s_in) {
#pragma unroll
      for (int j = 0; j < 64; ++j) s_out[(int64_t)j * kD] = S[j];
    }
    bool ok = true;
    float g_next = n_chunks > 0 ? gcs[0] : 0.f;           // g_C of chunk i - 1, fetched one iteration ahead
    for (int i = 0; i <= n_chunks && n_chunks > 0; ++i) {
      const float gC = g_next;
      if (i < n_chunks) g_next = gcs[i];
      // ---- state phase: after this block S is the state before chunk i ---------------------------
      if (i > 0) {
        ok = mbar_wait(&bar.s_done, (uint32_t)(i - 1) & 1u, abort_flag);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after();
        uint32_t d[64];
        tmem_ld32_nowait(lane_base + kColS + 64 * half, &d[0]);
        tmem_ld32_nowait(lane_base + kColS + 64 * half + 32, &d[32]);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 64; ++j) { reg_fence(d[j]); S[j] = fmaf(gC, S[j], __uint_as_float(d[j])); }
      }
      if (i < n_chunks) {                               // 16-bit copy of S^T: the A operand of MMA1a/b
        uint32_t w[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) w[j] = pack2<kBf16>(S[2 * j], S[2 * j + 1]);
        tmem_st32(lane_base + kColSb + 32 * half, w);
        tmem_st_wait();
        tc_fence_before();                                // also: the dS^T columns have been read, MMA2a may overwrite them
        __syncwarp();
        if (lane == 0) mbar_arrive(&bar.sb_ready);
      }
      // snapshot / final state: the state after i chunks
      if (i > 0 && snap_base != nullptr && (i % p.var.snap_chunks) == 0 && tok_base + (int64_t)i * kC <= tok_end) {
        float* dst = snap_base + (int64_t)(i / p.var.snap_chunks - 1) * p.H * kD * kD;
#pragma unroll
        for (int j = 0; j < 64; ++j) dst[(int64_t)j * kD] = S[j];
      }
      if (i == n_chunks && s_out != nullptr) {
#pragma unroll
        for (int j = 0; j < 64; ++j) s_out[(int64_t)j * kD] = S[j];
      }

      // ---- O^T of the previous chunk, one chunk behind: thread (v, half) holds rows p = 32*half .. +31 ----
      if (want_o && i > 0) {
        const int ci = i - 1, ob = ci & 1;
        ok = mbar_wait(&bar.o_done[ob], (uint32_t)(ci >> 1) & 1u, abort_flag);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after();
        uint32_t r[32];
        tmem_ld32(lane_base + kColO + ob * 64 + 32 * half, r);
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&bar.o_free[ob]);
        const int64_t t0 = tok_base + (int64_t)ci * kC + 32 * half;
        uint16_t* ocol = reinterpret_cast<uint16_t*>(p.o) + (t0 * p.H + h) * kD + row;
        const int n_ok = (int)min((int64_t)32, tok_end - t0);
#pragma unroll
        for (int j = 0; j < 32; ++j)
          if (j < n_ok) ocol[(int64_t)j * p.H * kD] = (uint16_t)(pack2<kBf16>(__uint_as_float(r[j]), 0.f) & 0xffffu);
      }

      // ---- U^T of this chunk: all 128 lanes, chunk rows 32*half .. +31 ------------------------------
      if (i < n_chunks) {
        const int s = i % kStages;
        const uint32_t ph = (uint32_t)(i / kStages) & 1u;
        ok = mbar_wait(&bar.u_full, (uint32_t)i & 1u, abort_flag);
        if (ok && !zero_u0) ok = mbar_wait(&bar.y_full[s], ph, abort_flag);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after();
        uint32_t r[32];
        tmem_ld32(lane_base + kColU + 32 * half, r);
        const uint8_t* u0_box = smem + s * kStageBytes + kA1Bytes + kKtBytes;
        uint32_t ow[16];
#pragma unroll
        for (int ch = 0; ch < 4; ++ch) {
          uint4 u0 = make_uint4(0u, 0u, 0u, 0u);
          if (!zero_u0) u0 = *reinterpret_cast<const uint4*>(u0_box + box_off(row, 4 * half + ch));
          const uint32_t uw[4] = {u0.x, u0.y, u0.z, u0.w};
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float2 f = unpack2<kBf16>(uw[e]);
            ow[4 * ch + e] = pack2<kBf16>(__uint_as_float(r[8 * ch + 2 * e]) + f.x, __uint_as_float(r[8 * ch + 2 * e + 1]) + f.y);
          }
        }
        tmem_st16(lane_base + kColUb + 16 * half, ow);
        tmem_st_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&bar.ub_ready);
      }

    }
  }

  tc_fence_before();
  __syncthreads();
  if (tid == 0 && s_abort) atomicExch(&g_scan_status, 1);
  if (warp == 1) tmem_dealloc(tbase, 512);
}

int make_record_maps(CUtensorMap* rec, CUtensorMap* rq, const uint8_t* recs, int is_bf16, int64_t n_records) {
  {
    const uint64_t rows = (uint64_t)n_records * kRecRows;
    const uint64_t dims[4] = {128, rows, 1, 1};
    const int64_t strides[3] = {128, (int64_t)rows * 128, (int64_t)rows * 128};
    const uint32_t box[4] = {64, 64, 1, 1};
    int rc = make_tmap_16bit_4d(rec, recs, is_bf16, dims, strides, box);
    if (rc != ATMA_OK) return rc;
  }
  const uint64_t rows = (uint64_t)n_records * kRecRowsRq;
  const uint64_t dims[4] = {64, rows, 1, 1};
  const int64_t strides[3] = {64, (int64_t)rows * 64, (int64_t)rows * 64};
  const uint32_t box[4] = {64, 64, 1, 1};
  return make_tmap_16bit_4d(rq, recs, is_bf16, dims, strides, box);
}

}  // namespace

int gated_delta_recur_sm100(const uint8_t* recs, const float* gcs, int is_bf16, int64_t n_records, const float* initial_state,
                            void* o, float* final_state, int Tlen, int H, int NC, int n_rec, const RecMap& map,
                            const VarLen& var, cudaStream_t st) {
  if (n_rec <= 0 || n_records <= 0) return ATMA_OK;
  if (n_records * kRecRowsRq >= (int64_t(1) << 31))
    return fail(ATMA_ERR_INVALID, "gated_delta_scan: %lld chunk records exceed the tensor-map row range", (long long)n_records);
  CUtensorMap mrec, mrq;
  int rc = make_record_maps(&mrec, &mrq, recs, is_bf16, n_records);
  if (rc != ATMA_OK) return rc;
  Params p{};
  p.gcs = gcs; p.initial_state = initial_state; p.o = o; p.final_state = final_state;
  p.Tlen = Tlen; p.H = H; p.NC = NC; p.is_bf16 = is_bf16; p.map = map; p.var = var;
  const dim3 grid(H, n_rec);
  if (is_bf16) {
    ATMA_CUDA_OK(cudaFuncSetAttribute(scan_recur_sm100_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes));
    scan_recur_sm100_kernel<true><<<grid, kThreads, kSmemBytes, st>>>(mrec, mrq, p);
  } else {
    ATMA_CUDA_OK(cudaFuncSetAttribute(scan_recur_sm100_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes));
    scan_recur_sm100_kernel<false><<<grid, kThreads, kSmemBytes, st>>>(mrec, mrq, p);
  }
  return launch_status("gated_delta_scan (recurrence, tcgen05)");
}

int scan_sm100_status_fetch_and_clear(int* out) {
  int v = 0, zero = 0;
  ATMA_CUDA_OK(cudaMemcpyFromSymbol(&v, g_scan_status, sizeof(int)));
  if (v != 0) ATMA_CUDA_OK(cudaMemcpyToSymbol(g_scan_status, &zero, sizeof(int)));
  *out = v;
  return ATMA_OK;
}

}  // namespace atma
