// Gated-delta chunked scan (chunk = 64 tokens), fp32 CUDA-core implementation.
//
// State per head S [dk][dv] ([K,V] layout).  With inclusive cumulative log-decay lg_p inside a
// chunk, g_p = exp(lg_p):
//   A[p,s]  = beta_p (g_p/g_s)(k_s.k_p), s < p          T = (I + A)^-1  (unit lower triangular)
//   W  = T diag(beta g) K      [C][dk]                  U0 = T diag(beta) V   [C][dv]
//   Qg = diag(g) Q             [C][dk]                  Kt = diag(g_C/g) K    [C][dk]
//   Rq[p,s] = (g_p/g_s)(k_s.q_p), s <= p
// and the chunk recurrence is three small products on the state:
//   U = U0 - W S ;   O = Qg S + Rq U ;   S <- g_C S + Kt^T U.
// Kernel 1 builds (W, Qg, Kt, U0, Rq, g_C) for every chunk in parallel (no dependence on S);
// kernel 2 walks the chunks of one (sequence, head, 32-column slice of S) in order - state
// columns are independent, so the dv/32 slices of a head run as separate CTAs.
#include "common.cuh"

namespace atma {

constexpr int kScanC = 64;            // tokens per chunk
constexpr int kScanThreads = 256;
constexpr int kScanSlice = 32;        // state columns per CTA in the sequential kernel

struct ScanScratch {                  // per-chunk record, in floats
  int dk, dv;
  __host__ __device__ int64_t w() const { return 0; }
  __host__ __device__ int64_t qg() const { return (int64_t)kScanC * dk; }
  __host__ __device__ int64_t kt() const { return (int64_t)2 * kScanC * dk; }
  __host__ __device__ int64_t u0() const { return (int64_t)3 * kScanC * dk; }
  __host__ __device__ int64_t rq() const { return u0() + (int64_t)kScanC * dv; }
  __host__ __device__ int64_t gc() const { return rq() + kScanC * kScanC; }
  __host__ __device__ int64_t stride() const { return gc() + 4; }
};

template <typename T>
__global__ void __launch_bounds__(kScanThreads)
scan_chunk_local_kernel(const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v,
                        const float* __restrict__ g, const float* __restrict__ beta,
                        float* __restrict__ scratch, int Tlen, int H, int Hkv, int dk, int dv,
                        int NC, int normalize_qk, float scale) {
  extern __shared__ float sm[];
  const int ld = dk + 1;
  float* Kn = sm;                                  // [C][dk+1]
  float* Qn = Kn + kScanC * ld;                    // [C][max(dk,dv)+1]  (later: beta * V)
  const int ldq = (dk > dv ? dk : dv) + 1;
  float* A = Qn + kScanC * ldq;                    // [C][C+1]
  float* Tm = A + kScanC * (kScanC + 1);           // [C][C+1]
  float* lg = Tm + kScanC * (kScanC + 1);          // [C]
  float* bt = lg + kScanC;                         // [C]
  float* eg = bt + kScanC;                         // [C]  exp(lg)
  const int ldA = kScanC + 1;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int c = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int t0 = c * kScanC;
  const int rows = min(kScanC, Tlen - t0);
  const ScanScratch lay{dk, dv};
  float* out = scratch + (((int64_t)b * H + h) * NC + c) * lay.stride();

  // rows of q, k (token stride H*dk), L2-normalised; rows past the end of the sequence are zero
  for (int r = warp; r < kScanC; r += kScanThreads / 32) {
    const bool ok = r < rows;
    const int64_t base = (((int64_t)b * Tlen + t0 + r) * H + h) * dk;
    const int64_t kbase = (((int64_t)b * Tlen + t0 + r) * Hkv + h / (H / Hkv)) * dk;
    float ks = 0.f, qs = 0.f;
    for (int d = lane; d < dk; d += 32) {
      const float kv = ok ? to_f32(k[kbase + d]) : 0.f, qv = ok ? to_f32(q[base + d]) : 0.f;
      Kn[r * ld + d] = kv; Qn[r * ldq + d] = qv;
      ks = fmaf(kv, kv, ks); qs = fmaf(qv, qv, qs);
    }
    ks = warp_sum(ks); qs = warp_sum(qs);
    const float kinv = normalize_qk ? 1.0f / fmaxf(sqrtf(ks), 1e-12f) : 1.0f;
    const float qinv = (normalize_qk ? 1.0f / fmaxf(sqrtf(qs), 1e-12f) : 1.0f) * scale;
    for (int d = lane; d < dk; d += 32) { Kn[r * ld + d] *= kinv; Qn[r * ldq + d] *= qinv; }
  }
  if (tid == 0) {
    float run = 0.f;
    for (int r = 0; r < kScanC; ++r) {
      const int64_t gi = ((int64_t)b * Tlen + t0 + r) * H + h;
      run += (r < rows) ? g[gi] : 0.f;
      lg[r] = run;
      eg[r] = __expf(run);
      bt[r] = (r < rows) ? beta[gi] : 0.f;
    }
  }
  __syncthreads();

  // A (strictly lower) and Rq (lower, self-inclusive)
  float* rq_out = out + lay.rq();
  for (int i = tid; i < kScanC * kScanC; i += kScanThreads) {
    const int s = i & (kScanC - 1), p = i >> 6;
    float kk = 0.f, qk = 0.f;
    if (s <= p) {
      const float* ks_ = Kn + s * ld; const float* kp_ = Kn + p * ld; const float* qp_ = Qn + p * ldq;
      for (int d = 0; d < dk; ++d) { const float x = ks_[d]; kk = fmaf(x, kp_[d], kk); qk = fmaf(x, qp_[d], qk); }
      const float ratio = __expf(lg[p] - lg[s]);
      kk *= ratio * bt[p]; qk *= ratio;
    }
    A[p * ldA + s] = (s < p) ? kk : 0.f;
    rq_out[p * kScanC + s] = (s <= p) ? qk : 0.f;
  }
  __syncthreads();

  // T = (I + A)^-1 by forward substitution: thread j owns column j of T.
  if (tid < kScanC) {
    const int j = tid;
    float col[kScanC];
#pragma unroll
    for (int p = 0; p < kScanC; ++p) {
      float acc = (p == j) ? 1.f : 0.f;
#pragma unroll
      for (int s = 0; s < p; ++s) acc = fmaf(-A[p * ldA + s], col[s], acc);
      col[p] = acc;
    }
#pragma unroll
    for (int p = 0; p < kScanC; ++p) Tm[p * ldA + j] = col[p];
  }
  __syncthreads();

  // W = T diag(beta g) K ; Qg ; Kt
  const float lgC = lg[kScanC - 1];
  for (int i = tid; i < kScanC * dk; i += kScanThreads) {
    const int p = i / dk, d = i - p * dk;
    float acc = 0.f;
    for (int s = 0; s <= p; ++s) acc = fmaf(Tm[p * ldA + s] * bt[s] * eg[s], Kn[s * ld + d], acc);
    out[lay.w() + i] = acc;
    out[lay.qg() + i] = eg[p] * Qn[p * ldq + d];
    out[lay.kt() + i] = __expf(lgC - lg[p]) * Kn[p * ld + d];
  }
  if (tid == 0) out[lay.gc()] = __expf(lgC);
  __syncthreads();

  // stage beta * V over the Qn buffer, then U0 = T (beta V)
  for (int i = tid; i < kScanC * dv; i += kScanThreads) {
    const int r = i / dv, d = i - r * dv;
    const int64_t base = (((int64_t)b * Tlen + t0 + r) * Hkv + h / (H / Hkv)) * dv;
    Qn[r * ldq + d] = (r < rows) ? bt[r] * to_f32(v[base + d]) : 0.f;
  }
  __syncthreads();
  for (int i = tid; i < kScanC * dv; i += kScanThreads) {
    const int p = i / dv, d = i - p * dv;
    float acc = 0.f;
    for (int s = 0; s <= p; ++s) acc = fmaf(Tm[p * ldA + s], Qn[s * ldq + d], acc);
    out[lay.u0() + i] = acc;
  }
}

template <typename T>
__global__ void __launch_bounds__(kScanThreads)
scan_sequential_kernel(const float* __restrict__ scratch, const float* __restrict__ initial_state,
                       T* __restrict__ o, float* __restrict__ final_state, int Tlen, int H, int dk,
                       int dv, int NC) {
  extern __shared__ float sm[];
  float* S = sm;                                   // [dk][32]
  float* Ws = S + dk * kScanSlice;                 // [C][dk]
  float* Qs = Ws + kScanC * dk;                    // [C][dk]
  float* Ks = Qs + kScanC * dk;                    // [C][dk]
  float* Us = Ks + kScanC * dk;                    // [C][32]
  float* Rq = Us + kScanC * kScanSlice;            // [C][C]

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  constexpr int NW = kScanThreads / 32;
  const int slice = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int col = slice * kScanSlice + lane;
  const bool col_ok = col < dv;
  const ScanScratch lay{dk, dv};
  const int64_t sbase = ((int64_t)b * H + h) * dk * dv;

  for (int kk = warp; kk < dk; kk += NW)
    S[kk * kScanSlice + lane] = (initial_state && col_ok) ? initial_state[sbase + (int64_t)kk * dv + col] : 0.f;
  __syncthreads();

  for (int c = 0; c < NC; ++c) {
    const float* rec = scratch + (((int64_t)b * H + h) * NC + c) * lay.stride();
    for (int i = tid; i < kScanC * dk; i += kScanThreads) {
      Ws[i] = rec[lay.w() + i]; Qs[i] = rec[lay.qg() + i]; Ks[i] = rec[lay.kt() + i];
    }
    for (int i = tid; i < kScanC * kScanC; i += kScanThreads) Rq[i] = rec[lay.rq() + i];
    const float gC = rec[lay.gc()];
    __syncthreads();

    // U = U0 - W S   (thread: column `lane`, rows warp, warp+8, ...)
    float qs[kScanC / NW];
#pragma unroll
    for (int i = 0; i < kScanC / NW; ++i) {
      const int p = warp + NW * i;
      float u = col_ok ? rec[lay.u0() + p * dv + col] : 0.f;
      float r = 0.f;
      const float* wr = Ws + p * dk; const float* qr = Qs + p * dk;
      for (int kk = 0; kk < dk; ++kk) {
        const float sv = S[kk * kScanSlice + lane];
        u = fmaf(-wr[kk], sv, u);
        r = fmaf(qr[kk], sv, r);
      }
      Us[p * kScanSlice + lane] = u;
      qs[i] = r;
    }
    __syncthreads();
    // O = Qg S + Rq U
    const int t0 = c * kScanC;
#pragma unroll
    for (int i = 0; i < kScanC / NW; ++i) {
      const int p = warp + NW * i;
      float r = qs[i];
      const float* rr = Rq + p * kScanC;
      for (int s = 0; s <= p; ++s) r = fmaf(rr[s], Us[s * kScanSlice + lane], r);
      if (t0 + p < Tlen && col_ok) o[(((int64_t)b * Tlen + t0 + p) * H + h) * dv + col] = from_f32<T>(r);
    }
    // S <- gC S + Kt^T U
    for (int kk = warp; kk < dk; kk += NW) {
      float acc = gC * S[kk * kScanSlice + lane];
      for (int s = 0; s < kScanC; ++s) acc = fmaf(Ks[s * dk + kk], Us[s * kScanSlice + lane], acc);
      S[kk * kScanSlice + lane] = acc;
    }
    __syncthreads();
  }
  if (final_state && col_ok)
    for (int kk = warp; kk < dk; kk += NW) final_state[sbase + (int64_t)kk * dv + col] = S[kk * kScanSlice + lane];
}

// tensor-core version for 16-bit inputs with d_k = d_v = 128 (gated_delta_scan_mma.cu)
bool gated_delta_scan_mma_supported(int dtype, int dk, int dv);
int64_t gated_delta_scan_mma_scratch_bytes(int B, int T, int H);
int gated_delta_scan_mma(const void* q, const void* k, const void* v, int dtype, const float* g, const float* beta,
                         const float* initial_state, void* o, float* final_state, void* scratch, int B, int T, int H,
                         int Hkv, int normalize_qk, float scale, int segments, cudaStream_t st);

int gated_delta_scan_mma_factors(const void* q, const void* k, const void* v, int dtype, const float* g,
                                 const float* beta, void* scratch, int B, int T, int H, int Hkv, int normalize_qk,
                                 float scale, cudaStream_t st);
int gated_delta_scan_mma_recur(void* scratch, int dtype, int B, int T, int H, int n_rec, const int* rec_of,
                               const int* zero_u0, const float* initial_state, void* o, float* final_state,
                               cudaStream_t st);
int64_t gated_delta_scan_mma_varlen_scratch_bytes(int64_t total_tokens, int n_seqs, int H);
int gated_delta_scan_mma_varlen(const void* q, const void* k, const void* v, int dtype, const float* g, const float* beta,
                                const int32_t* cu_seqlens, int n_seqs, int64_t total_tokens, const float* initial_state,
                                float* final_state, float* state_table, int64_t slot_stride, const int64_t* slots,
                                const int32_t* has_initial, void* o, void* scratch, int H, int Hkv, int normalize_qk,
                                float scale, float* snapshots, const int32_t* snap_offsets, int snap_chunks,
                                cudaStream_t st);

}  // namespace atma

using namespace atma;

extern "C" int atma_gated_delta_scan_factors(const void* q, const void* k, const void* v, int dtype, const float* g,
                                             const float* beta, void* scratch, int B, int T, int H, int Hkv, int dk,
                                             int dv, int normalize_qk, float scale, void* stream) {
  ATMA_REQUIRE(gated_delta_scan_mma_supported(dtype, dk, dv),
               "gated_delta_scan_factors: needs 16-bit inputs with dk = dv = 128 (got dtype %d, dk %d, dv %d)", dtype, dk, dv);
  ATMA_REQUIRE(B > 0 && T > 0 && H > 0 && Hkv > 0 && H % Hkv == 0, "gated_delta_scan_factors: bad shape");
  ATMA_REQUIRE(scratch != nullptr && (uintptr_t)scratch % 256 == 0 && (uintptr_t)q % 16 == 0 && (uintptr_t)k % 16 == 0 &&
                   (uintptr_t)v % 16 == 0, "gated_delta_scan_factors: scratch must be 256-byte and inputs 16-byte aligned");
  return gated_delta_scan_mma_factors(q, k, v, dtype, g, beta, scratch, B, T, H, Hkv, normalize_qk, scale, (cudaStream_t)stream);
}

extern "C" int atma_gated_delta_scan_recur(void* scratch, int dtype, int B, int T, int H, int dk, int dv, int n_rec,
                                           const int* rec_of, const int* zero_u0, const float* initial_state, void* o,
                                           float* final_state, void* stream) {
  ATMA_REQUIRE(gated_delta_scan_mma_supported(dtype, dk, dv), "gated_delta_scan_recur: needs 16-bit, dk = dv = 128");
  ATMA_REQUIRE(scratch != nullptr && B > 0 && T > 0 && H > 0, "gated_delta_scan_recur: bad arguments");
  return gated_delta_scan_mma_recur(scratch, dtype, B, T, H, n_rec, rec_of, zero_u0, initial_state, o, final_state,
                                    (cudaStream_t)stream);
}

extern "C" int64_t atma_gated_delta_scan_varlen_scratch_bytes(int64_t total_tokens, int n_seqs, int H, int dk, int dv) {
  if (!gated_delta_scan_mma_supported(ATMA_BF16, dk, dv) || total_tokens < 0 || n_seqs < 0) return 0;
  return gated_delta_scan_mma_varlen_scratch_bytes(total_tokens, n_seqs, H);
}

static int scan_varlen_impl(const void* q, const void* k, const void* v, int dtype, const float* g,
                                            const float* beta, const int32_t* cu_seqlens, int n_seqs,
                                            int64_t total_tokens, const float* initial_state, float* final_state,
                                            float* state_table, int64_t slot_stride, const int64_t* slots,
                                            const int32_t* has_initial, void* o, void* scratch, int H, int Hkv, int dk,
                                            int dv, int normalize_qk, float scale, float* snapshots,
                                            const int32_t* snap_offsets, int snap_every_tokens, void* stream) {
  ATMA_REQUIRE(gated_delta_scan_mma_supported(dtype, dk, dv),
               "gated_delta_scan_varlen: needs 16-bit inputs with dk = dv = 128 (got dtype %d, dk %d, dv %d)", dtype, dk, dv);
  ATMA_REQUIRE(n_seqs >= 0 && total_tokens >= 0 && H > 0 && Hkv > 0 && H % Hkv == 0, "gated_delta_scan_varlen: bad shape");
  ATMA_REQUIRE(total_tokens / kScanC + n_seqs < (1 << 30), "gated_delta_scan_varlen: too many chunks");
  ATMA_REQUIRE(n_seqs <= 65535, "gated_delta_scan_varlen: at most 65535 sequences per call (got %d)", n_seqs);
  ATMA_REQUIRE(snapshots == nullptr || (snap_offsets != nullptr && snap_every_tokens > 0 && snap_every_tokens % kScanC == 0),
               "gated_delta_scan_varlen: snapshots need offsets and a spacing that is a multiple of %d tokens", kScanC);
  if (n_seqs == 0) return ATMA_OK;
  ATMA_REQUIRE(cu_seqlens != nullptr, "gated_delta_scan_varlen: cu_seqlens is required");
  ATMA_REQUIRE(state_table == nullptr || slots != nullptr, "gated_delta_scan_varlen: a state table needs slots");
  ATMA_REQUIRE(state_table == nullptr || (initial_state == nullptr && final_state == nullptr),
               "gated_delta_scan_varlen: pass either a slot-indexed state table or dense state arrays, not both");
  ATMA_REQUIRE(scratch != nullptr && (uintptr_t)scratch % 256 == 0 && (uintptr_t)q % 16 == 0 && (uintptr_t)k % 16 == 0 &&
                   (uintptr_t)v % 16 == 0, "gated_delta_scan_varlen: scratch must be 256-byte and inputs 16-byte aligned");
  return gated_delta_scan_mma_varlen(q, k, v, dtype, g, beta, cu_seqlens, n_seqs, total_tokens, initial_state, final_state,
                                     state_table, slot_stride, slots, has_initial, o, scratch, H, Hkv, normalize_qk, scale,
                                     snapshots, snap_offsets, snapshots ? snap_every_tokens / kScanC : 0, (cudaStream_t)stream);
}

extern "C" int atma_gated_delta_scan_varlen(const void* q, const void* k, const void* v, int dtype, const float* g,
                                            const float* beta, const int32_t* cu_seqlens, int n_seqs,
                                            int64_t total_tokens, const float* initial_state, float* final_state,
                                            float* state_table, int64_t slot_stride, const int64_t* slots,
                                            const int32_t* has_initial, void* o, void* scratch, int H, int Hkv, int dk,
                                            int dv, int normalize_qk, float scale, void* stream) {
  return scan_varlen_impl(q, k, v, dtype, g, beta, cu_seqlens, n_seqs, total_tokens, initial_state, final_state, state_table,
                          slot_stride, slots, has_initial, o, scratch, H, Hkv, dk, dv, normalize_qk, scale, nullptr, nullptr, 0,
                          stream);
}

extern "C" int atma_gated_delta_scan_varlen_snapshots(const void* q, const void* k, const void* v, int dtype, const float* g,
                                                      const float* beta, const int32_t* cu_seqlens, int n_seqs,
                                                      int64_t total_tokens, float* state_table, int64_t slot_stride,
                                                      const int64_t* slots, const int32_t* has_initial, void* o,
                                                      void* scratch, int H, int Hkv, int dk, int dv, int normalize_qk,
                                                      float scale, float* snapshots, const int32_t* snap_offsets,
                                                      int snap_every_tokens, void* stream) {
  ATMA_REQUIRE(snapshots != nullptr, "gated_delta_scan_varlen_snapshots: the snapshot buffer is required");
  return scan_varlen_impl(q, k, v, dtype, g, beta, cu_seqlens, n_seqs, total_tokens, nullptr, nullptr, state_table, slot_stride,
                          slots, has_initial, o, scratch, H, Hkv, dk, dv, normalize_qk, scale, snapshots, snap_offsets,
                          snap_every_tokens, stream);
}

extern "C" int64_t atma_gated_delta_scan_scratch_bytes(int B, int T, int H, int dk, int dv) {
  const int NC = (T + kScanC - 1) / kScanC;
  const ScanScratch lay{dk, dv};
  const int64_t fp32_path = (int64_t)B * H * NC * lay.stride() * (int64_t)sizeof(float);
  const int64_t mma_path = gated_delta_scan_mma_scratch_bytes(B, T, H);
  return fp32_path > mma_path ? fp32_path : mma_path;
}

extern "C" int atma_gated_delta_scan(const void* q, const void* k, const void* v, int dtype,
                                     const float* g, const float* beta, const float* initial_state,
                                     void* o, float* final_state, void* scratch, int B, int T, int H,
                                     int Hkv, int dk, int dv, int normalize_qk, float scale,
                                     void* stream) {
  return atma_gated_delta_scan_segmented(q, k, v, dtype, g, beta, initial_state, o, final_state, scratch, B, T, H, Hkv, dk, dv,
                                         normalize_qk, scale, 0, stream);
}

extern "C" int atma_gated_delta_scan_segmented(const void* q, const void* k, const void* v, int dtype,
                                               const float* g, const float* beta, const float* initial_state,
                                               void* o, float* final_state, void* scratch, int B, int T, int H,
                                               int Hkv, int dk, int dv, int normalize_qk, float scale,
                                               int segments, void* stream) {
  ATMA_REQUIRE(segments >= 0 && segments <= 16, "gated_delta_scan: segments=%d outside 0..16", segments);
  ATMA_REQUIRE(dtype_ok(dtype), "gated_delta_scan: unsupported dtype %d", dtype);
  ATMA_REQUIRE(dk >= 1 && dk <= 128 && dv >= 1 && dv <= 128, "gated_delta_scan: dk=%d dv=%d outside 1..128", dk, dv);
  ATMA_REQUIRE(B >= 0 && T >= 0 && H > 0, "gated_delta_scan: bad shape");
  ATMA_REQUIRE(Hkv > 0 && H % Hkv == 0, "gated_delta_scan: H=%d is not a multiple of Hkv=%d", H, Hkv);
  ATMA_REQUIRE(scratch != nullptr || B * T == 0, "gated_delta_scan: scratch is required");
  cudaStream_t st = (cudaStream_t)stream;
  if (B == 0) return ATMA_OK;
  if (T == 0) {                                     // nothing to scan: the state passes through
    if (final_state && initial_state)
      ATMA_CUDA_OK(cudaMemcpyAsync(final_state, initial_state, sizeof(float) * (size_t)B * H * dk * dv,
                                   cudaMemcpyDeviceToDevice, st));
    else if (final_state)
      ATMA_CUDA_OK(cudaMemsetAsync(final_state, 0, sizeof(float) * (size_t)B * H * dk * dv, st));
    return ATMA_OK;
  }
  if (gated_delta_scan_mma_supported(dtype, dk, dv) && ((uintptr_t)q % 16 == 0) && ((uintptr_t)k % 16 == 0) &&
      ((uintptr_t)v % 16 == 0) && ((uintptr_t)scratch % 256 == 0))
    return gated_delta_scan_mma(q, k, v, dtype, g, beta, initial_state, o, final_state, scratch, B, T, H, Hkv,
                                normalize_qk, scale, segments, st);
  const int NC = (T + kScanC - 1) / kScanC;
  const int ldq = (dk > dv ? dk : dv) + 1;
  const size_t smem1 = sizeof(float) * ((size_t)kScanC * (dk + 1) + (size_t)kScanC * ldq +
                                        2 * (size_t)kScanC * (kScanC + 1) + 3 * kScanC);
  const size_t smem2 = sizeof(float) * ((size_t)dk * kScanSlice + 3 * (size_t)kScanC * dk +
                                        (size_t)kScanC * kScanSlice + (size_t)kScanC * kScanC);
  int rc = ATMA_OK;
  ATMA_DISPATCH_DTYPE(dtype, TT, {
    auto k1 = scan_chunk_local_kernel<TT>;
    auto k2 = scan_sequential_kernel<TT>;
    ATMA_CUDA_OK(cudaFuncSetAttribute(k1, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem1));
    ATMA_CUDA_OK(cudaFuncSetAttribute(k2, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem2));
    k1<<<dim3(NC, H, B), kScanThreads, smem1, st>>>((const TT*)q, (const TT*)k, (const TT*)v, g, beta,
                                                     (float*)scratch, T, H, Hkv, dk, dv, NC, normalize_qk, scale);
    rc = launch_status("gated_delta_scan (chunk-local)");
    if (rc == ATMA_OK) {
      k2<<<dim3((dv + kScanSlice - 1) / kScanSlice, H, B), kScanThreads, smem2, st>>>(
          (const float*)scratch, initial_state, (TT*)o, final_state, T, H, dk, dv, NC);
      rc = launch_status("gated_delta_scan (sequential)");
    }
  });
  return rc;
}
