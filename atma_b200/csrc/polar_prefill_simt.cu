// Polar Attention prefill on the CUDA cores, fp32 arithmetic throughout.
//
// This is the path for fp32 tensors (the reference's "ieee" precision, pinned at 1e-4) and
// for head sizes / layouts the tensor-core tile kernel does not take.  It streams key tiles
// with running (m, L, Q2, S) per query row, supports GQA without expanded K/V, arbitrary
// per-query key counts, a sliding window, a packed ragged batch, and carry-in / carry-out
// of the running statistics for a ring pass over remote K/V blocks.
//
// CTA = 8 warps x 4 query rows; key tile = 32 rows staged in shared memory as fp32.
// Scores: lane j owns key j of the tile (K rows padded to dk+1 floats: conflict-free),
// q rows are shared-memory broadcasts.  P.V: lane owns columns lane, lane+32, ...; p_j
// arrives by shuffle.
#include "common.cuh"
#include "polar_prefill.cuh"

namespace atma {

constexpr int kSimtWarps = 8;
constexpr int kSimtRowsPerWarp = 4;
constexpr int kSimtBM = kSimtWarps * kSimtRowsPerWarp;   // 32 query rows per CTA
constexpr int kSimtBN = 32;                              // keys per tile
constexpr float kNegBig = -1e38f;

template <typename T, int DK>
__global__ void __launch_bounds__(kSimtWarps * 32)
polar_prefill_simt_kernel(const atma_polar_prefill_args a) {
  constexpr int NSLOT = DK / 32;
  extern __shared__ float smem[];
  float* Qs = smem;                                  // [BM][DK]
  float* Ks = Qs + kSimtBM * DK;                     // [BN][DK+1]
  float* Vs = Ks + kSimtBN * (DK + 1);               // [BN][DK]
  __shared__ float s_nmin, s_nmax;
  __shared__ float s_wmin[kSimtWarps], s_wmax[kSimtWarps];

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int h = blockIdx.y, b = blockIdx.z;
  const int kvh = h / (a.H / a.Hkv);

  // ---- which query rows / which sequence ----------------------------------------------------
  int q_row0, seq_row0 = 0, q_limit, k_limit;
  const bool packed = a.n_tiles > 0;
  if (packed) {
    const int t = blockIdx.x / (128 / kSimtBM), sub = blockIdx.x % (128 / kSimtBM);
    seq_row0 = a.tile_seq_start[t];
    q_row0 = a.tile_q_start[t] + sub * kSimtBM;
    q_limit = a.tile_seq_len[t];
    k_limit = q_limit;
  } else {
    q_row0 = blockIdx.x * kSimtBM;
    q_limit = a.Tq;
    k_limit = a.Tk;
  }
  if (q_row0 >= q_limit) return;

  const T* qp = (const T*)a.q + b * a.q_sb + h * a.q_sh;
  const T* kp = (const T*)a.k + b * a.k_sb + kvh * a.k_sh;
  const T* vp = (const T*)a.v + b * a.v_sb + kvh * a.v_sh;

  // ---- per-row scalars ----------------------------------------------------------------------
  float n_i[kSimtRowsPerWarp], sc[kSimtRowsPerWarp], temp[kSimtRowsPerWarp];
  float m[kSimtRowsPerWarp], L[kSimtRowsPerWarp], Q2[kSimtRowsPerWarp];
  float acc[kSimtRowsPerWarp][NSLOT];
  bool row_ok[kSimtRowsPerWarp];
  const float spg = a.spg[h];
  const float inv_sqrt_dk = rsqrtf((float)DK);
  float wmin = 3.0e38f, wmax = -1.0f;
#pragma unroll
  for (int i = 0; i < kSimtRowsPerWarp; ++i) {
    const int r = q_row0 + warp * kSimtRowsPerWarp + i;
    row_ok[i] = r < q_limit;
    float n = 0.f;
    if (row_ok[i]) n = packed ? (float)(r + 1) : (a.n_keys ? a.n_keys[r] : a.n_base + (float)(r + 1));
    n_i[i] = n;
    const float nc = fmaxf(a.window > 0 ? fminf(n, (float)a.window) : n, 1.0f);
    temp[i] = 1.0f + spg * logf(nc);
    sc[i] = temp[i] * inv_sqrt_dk;
    if (row_ok[i]) { wmin = fminf(wmin, n); wmax = fmaxf(wmax, n); }
    const int64_t srow = ((int64_t)b * a.H + h) * a.Tq + r;     // dense stats index
    if (a.stats_in_m != nullptr && row_ok[i]) {
      m[i] = a.stats_in_m[srow]; L[i] = a.stats_in_l[srow]; Q2[i] = a.stats_in_q2[srow];
#pragma unroll
      for (int s = 0; s < NSLOT; ++s) acc[i][s] = a.stats_in_s[srow * DK + lane + 32 * s];
    } else {
      m[i] = kNegBig; L[i] = 0.f; Q2[i] = 0.f;
#pragma unroll
      for (int s = 0; s < NSLOT; ++s) acc[i][s] = 0.f;
    }
  }
  if (lane == 0) { s_wmin[warp] = wmin; s_wmax[warp] = wmax; }

  // ---- stage the Q rows (fp32) ----------------------------------------------------------------
  for (int i = tid; i < kSimtBM * DK; i += blockDim.x) {
    const int r = i / DK, d = i - r * DK;
    const int row = q_row0 + r;
    Qs[i] = row < q_limit ? to_f32(qp[(int64_t)(seq_row0 + row) * a.q_st + d]) : 0.f;
  }
  __syncthreads();
  if (tid == 0) {
    float lo = 3.0e38f, hi = -1.0f;
    for (int w = 0; w < kSimtWarps; ++w) { lo = fminf(lo, s_wmin[w]); hi = fmaxf(hi, s_wmax[w]); }
    s_nmin = lo; s_nmax = hi;
  }
  __syncthreads();

  // ---- key range this CTA must visit: tiles wholly invisible to every row are skipped ---------
  const float koff = (float)a.key_offset;
  int j_hi = (int)fminf((float)k_limit, ceilf(s_nmax - koff));
  j_hi = max(j_hi, 0);
  int j_lo = 0;
  if (a.window > 0) {
    const float first = s_nmin - (float)a.window - koff;
    if (first > 0.f) j_lo = ((int)first / kSimtBN) * kSimtBN;
  }

  for (int j0 = j_lo; j0 < j_hi; j0 += kSimtBN) {
    // stage K and V tile
    for (int i = tid; i < kSimtBN * DK; i += blockDim.x) {
      const int j = i / DK, d = i - j * DK;
      const int kr = j0 + j;
      float kv = 0.f, vv = 0.f;
      if (kr < k_limit) {
        kv = to_f32(kp[(int64_t)(seq_row0 + kr) * a.k_st + d]);
        vv = to_f32(vp[(int64_t)(seq_row0 + kr) * a.v_st + d]);
      }
      Ks[j * (DK + 1) + d] = kv;
      Vs[j * DK + d] = vv;
    }
    __syncthreads();

    float s[kSimtRowsPerWarp];
#pragma unroll
    for (int i = 0; i < kSimtRowsPerWarp; ++i) s[i] = 0.f;
    const float* krow = Ks + lane * (DK + 1);
    const float* qrow = Qs + warp * kSimtRowsPerWarp * DK;
#pragma unroll 8
    for (int d = 0; d < DK; ++d) {
      const float kv = krow[d];
#pragma unroll
      for (int i = 0; i < kSimtRowsPerWarp; ++i) s[i] = fmaf(qrow[i * DK + d], kv, s[i]);
    }
    const float pos = (float)(j0 + lane) + koff;
    const bool in_range = (j0 + lane) < k_limit;
#pragma unroll
    for (int i = 0; i < kSimtRowsPerWarp; ++i) {
      bool valid = in_range && row_ok[i] && pos < n_i[i];
      if (a.window > 0) valid = valid && pos >= n_i[i] - (float)a.window;
      const float av = valid ? s[i] * sc[i] : kNegBig;
      const float m_new = fmaxf(m[i], warp_max(av));
      const float alpha = expf(m[i] - m_new);
      const float p = valid ? expf(av - m_new) : 0.f;
      L[i] = L[i] * alpha + warp_sum(p);
      Q2[i] = Q2[i] * alpha * alpha + warp_sum(p * p);
      m[i] = m_new;
#pragma unroll
      for (int sl = 0; sl < NSLOT; ++sl) acc[i][sl] *= alpha;
#pragma unroll 8
      for (int j = 0; j < kSimtBN; ++j) {
        const float pj = __shfl_sync(0xffffffffu, p, j);
#pragma unroll
        for (int sl = 0; sl < NSLOT; ++sl) acc[i][sl] = fmaf(pj, Vs[j * DK + lane + 32 * sl], acc[i][sl]);
      }
    }
    __syncthreads();
  }

  // ---- epilogue ---------------------------------------------------------------------------------
#pragma unroll
  for (int i = 0; i < kSimtRowsPerWarp; ++i) {
    if (!row_ok[i]) continue;                                   // warp-uniform
    const int r = q_row0 + warp * kSimtRowsPerWarp + i;
    const int64_t srow = ((int64_t)b * a.H + h) * a.Tq + r;
    if (!a.finalize) {
      if (lane == 0) { a.stats_out_m[srow] = m[i]; a.stats_out_l[srow] = L[i]; a.stats_out_q2[srow] = Q2[i]; }
#pragma unroll
      for (int sl = 0; sl < NSLOT; ++sl) a.stats_out_s[srow * DK + lane + 32 * sl] = acc[i][sl];
      continue;
    }
    const float nc = fmaxf(a.window > 0 ? fminf(n_i[i], (float)a.window) : n_i[i], 1.0f);
    const float a_n = temp[i] * (a.null_base[h] + a.sps[h] * sqrtf(logf(nc + 1.0f)));
    const float m_new = fmaxf(m[i], a_n);
    const float alpha = expf(m[i] - m_new);
    const float Lf = L[i] * alpha, Q2f = Q2[i] * alpha * alpha;
    const float p_n = expf(a_n - m_new);
    const float Z = Lf + p_n;
    float sv[NSLOT], sq = 0.f;
#pragma unroll
    for (int sl = 0; sl < NSLOT; ++sl) {
      sv[sl] = acc[i][sl] * alpha + p_n * a.v_null[h * DK + lane + 32 * sl];
      sq = fmaf(sv[sl], sv[sl], sq);
    }
    const float inv = 1.0f / fmaxf(sqrtf(warp_sum(sq)), a.eps);
    T* cp = (T*)a.c + b * a.c_sb + h * a.c_sh + (int64_t)(seq_row0 + r) * a.c_st;
#pragma unroll
    for (int sl = 0; sl < NSLOT; ++sl) cp[lane + 32 * sl] = from_f32<T>(sv[sl] * inv);
    if (lane == 0) {
      const float n_eff = Lf * Lf / fmaxf(Q2f, 1e-30f);
      const float m_eff = n_eff * (Lf / fmaxf(Z, a.eps));
      ((T*)a.mag)[b * a.mag_sb + h * a.mag_sh + (int64_t)(seq_row0 + r) * a.mag_st] =
          from_f32<T>(tanhf(a.beta[h] * log1pf(m_eff)));
    }
  }
}

template <typename T, int DK>
int launch_simt(const atma_polar_prefill_args& a, cudaStream_t st) {
  const size_t smem = sizeof(float) * (kSimtBM * DK + kSimtBN * (DK + 1) + kSimtBN * DK);
  auto kern = polar_prefill_simt_kernel<T, DK>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return fail(ATMA_ERR_CUDA, "polar_prefill: smem opt-in failed: %s", cudaGetErrorString(e));
  dim3 grid(a.n_tiles > 0 ? a.n_tiles * (128 / kSimtBM) : (a.Tq + kSimtBM - 1) / kSimtBM, a.H, a.B);
  kern<<<grid, kSimtWarps * 32, smem, st>>>(a);
  return launch_status("polar_prefill (fp32 CUDA-core kernel)");
}

int polar_prefill_simt(const atma_polar_prefill_args& a, cudaStream_t st) {
  int rc = ATMA_OK;
  ATMA_DISPATCH_DTYPE(a.dtype, T, {
    switch (a.dk) {
      case 32: rc = launch_simt<T, 32>(a, st); break;
      case 64: rc = launch_simt<T, 64>(a, st); break;
      case 128: rc = launch_simt<T, 128>(a, st); break;
      case 256: rc = launch_simt<T, 256>(a, st); break;
      default: rc = fail(ATMA_ERR_UNSUPPORTED, "polar_prefill: head_dim %d not in {32,64,128,256}", a.dk);
    }
  });
  return rc;
}

}  // namespace atma
