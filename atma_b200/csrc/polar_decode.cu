// Paged Polar decode: one query token per sequence over its paged K/V context.
//
// Bandwidth-bound (every cached K and V byte is read once per step, once per GQA group),
// so the design is about HBM, not tensor cores:
//   * grid = (n_splits, Hkv, B): each (sequence, KV head) context is cut into n_splits key
//     ranges so that B*Hkv*n_splits CTAs cover the 148 SMs several times over; all G = H/Hkv
//     query heads of the group share each loaded K/V row;
//   * a key row (dk elements) is read by dk/8 adjacent lanes with one 16-byte load each, so
//     a warp instruction covers whole contiguous rows; kUnroll rows of K and of V are in
//     flight per lane before any arithmetic; the page table is read once per row;
//   * scores are reduced with xor-shuffles inside the dk/8-lane group; each lane group keeps
//     its own running (m, L, Q2, S) and the groups are merged once at the end of the CTA;
//   * partial statistics go to caller scratch, and a second kernel merges the splits with the
//     Polar rule (L and S scale by e^{m_i-M}, Q2 by its square), folds the null sink once and
//     writes c and mag.
// Launch shapes depend only on host-side arguments, loop bounds come from context_lens on the
// device: the pair of launches is CUDA-graph capturable.
#include "common.cuh"

namespace atma {

constexpr int kDecWarps = 4;
constexpr int kDecUnroll = 4;
constexpr int kDecMaxG = 8;
constexpr float kNegBig = -1e38f;

template <typename T>
__device__ __forceinline__ void load8(const T* p, float (&f)[8]);
template <>
__device__ __forceinline__ void load8<float>(const float* p, float (&f)[8]) {
  float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
  f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
}
template <>
__device__ __forceinline__ void load8<__nv_bfloat16>(const __nv_bfloat16* p, float (&f)[8]) {
  uint4 r = *reinterpret_cast<const uint4*>(p);
  const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {           // bf16 -> fp32 is a 16-bit shift
    f[2 * i] = __uint_as_float(w[i] << 16);
    f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
  }
}
template <>
__device__ __forceinline__ void load8<__half>(const __half* p, float (&f)[8]) {
  uint4 r = *reinterpret_cast<const uint4*>(p);
  const __half2* h = reinterpret_cast<const __half2*>(&r);
#pragma unroll
  for (int i = 0; i < 4; ++i) { float2 t = __half22float2(h[i]); f[2 * i] = t.x; f[2 * i + 1] = t.y; }
}

// scratch layout (floats): stats [B][H][n_splits][4] = (m, L, Q2, pad) then S [B][H][n_splits][dk]
__host__ __device__ inline int64_t dec_stats_off(int64_t bh, int split, int n_splits) {
  return (bh * n_splits + split) * 4;
}

template <typename T, int DK, int GMAX>
__global__ void __launch_bounds__(kDecWarps * 32)
polar_decode_split_kernel(const T* __restrict__ q, const T* __restrict__ k_cache,
                          const T* __restrict__ v_cache, const int32_t* __restrict__ block_tables,
                          int64_t bt_stride, const int32_t* __restrict__ context_lens, const int32_t* __restrict__ temp_lens,
                          const float* __restrict__ spg, float* __restrict__ scratch, int B, int H,
                          int Hkv, int block_size, int max_blocks, int num_blocks, int n_splits,
                          int window) {
  constexpr int LPR = DK / 8;              // lanes per key row
  constexpr int GPW = 32 / LPR;            // key rows per warp instruction
  constexpr int ROWS_PER_STEP = GPW * kDecWarps;
  const int split = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
  const int G = H / Hkv;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int sub = lane % LPR, grp = lane / LPR;
  const int d0 = sub * 8;

  int n = context_lens[b];
  n = max(0, min(n, max_blocks * block_size));
  const int lo_w = window > 0 ? max(n - window, 0) : 0;
  const int span = n - lo_w;
  int chunk = (span + n_splits - 1) / n_splits;
  chunk = (chunk + ROWS_PER_STEP - 1) / ROWS_PER_STEP * ROWS_PER_STEP;
  const int lo = lo_w + split * chunk;
  const int hi = min(lo + chunk, n);

  float* stats = scratch;
  float* sacc = scratch + (int64_t)B * H * n_splits * 4;

  if (lo >= hi) {                          // empty range: neutral partial
    for (int g = warp; g < G; g += kDecWarps) {
      const int64_t bh = (int64_t)b * H + kvh * G + g;
      if (lane == 0) {
        float4 z = make_float4(kNegBig, 0.f, 0.f, 0.f);
        *reinterpret_cast<float4*>(stats + dec_stats_off(bh, split, n_splits)) = z;
      }
      for (int d = lane; d < DK; d += 32) sacc[(bh * n_splits + split) * DK + d] = 0.f;
    }
    return;
  }

  const int nt = temp_lens != nullptr ? temp_lens[b] : n;      // the whole context sets the temperature
  const float nf = fmaxf(window > 0 ? fminf((float)nt, (float)window) : (float)nt, 1.0f);
  const float logn = logf(nf);
  const float inv_sqrt_dk = rsqrtf((float)DK);

  float qr[GMAX][8], acc[GMAX][8], m[GMAX], L[GMAX], Q2[GMAX];
#pragma unroll
  for (int g = 0; g < GMAX; ++g) {
    m[g] = kNegBig; L[g] = 0.f; Q2[g] = 0.f;
#pragma unroll
    for (int e = 0; e < 8; ++e) { acc[g][e] = 0.f; qr[g][e] = 0.f; }
    if (g < G) {
      const int h = kvh * G + g;
      const float sc = (1.0f + spg[h] * logn) * inv_sqrt_dk;   // temperature folded into q
      float t[8];
      load8<T>(q + ((int64_t)b * H + h) * DK + d0, t);
#pragma unroll
      for (int e = 0; e < 8; ++e) qr[g][e] = t[e] * sc;
    }
  }

  const int64_t row_stride = (int64_t)Hkv * DK;
  const int32_t* bt = block_tables + b * bt_stride;

  // The loop bound is warp-uniform (the shuffles below need all 32 lanes); a lane group whose
  // row falls past `hi` carries ok = false.
  for (int base0 = lo + warp * GPW; base0 < hi; base0 += ROWS_PER_STEP * kDecUnroll) {
    const int base = base0 + grp;
    float kf[kDecUnroll][8], vf[kDecUnroll][8];
    bool ok[kDecUnroll];
#pragma unroll
    for (int u = 0; u < kDecUnroll; ++u) {
      const int pos = base + u * ROWS_PER_STEP;
      ok[u] = pos < hi;
      if (ok[u]) {
        const int blk = pos / block_size;
        int phys = bt[blk];
        phys = min(max(phys, 0), num_blocks - 1);             // never dereference a bad page id
        const int64_t off = ((int64_t)phys * block_size + (pos - blk * block_size)) * row_stride +
                            (int64_t)kvh * DK + d0;
        load8<T>(k_cache + off, kf[u]);
        load8<T>(v_cache + off, vf[u]);
      }
    }
    float a[kDecUnroll][GMAX];
#pragma unroll
    for (int u = 0; u < kDecUnroll; ++u) {
#pragma unroll
      for (int g = 0; g < GMAX; ++g) {
        if (g < G) {
          float s = 0.f;
          if (ok[u]) {
#pragma unroll
            for (int e = 0; e < 8; ++e) s = fmaf(qr[g][e], kf[u][e], s);
          }
#pragma unroll
          for (int o = LPR / 2; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
          a[u][g] = ok[u] ? s : kNegBig;
        }
      }
    }
#pragma unroll
    for (int g = 0; g < GMAX; ++g) {
      if (g < G) {
        float mx = m[g];
#pragma unroll
        for (int u = 0; u < kDecUnroll; ++u) mx = fmaxf(mx, a[u][g]);
        const float alpha = __expf(m[g] - mx);
        float ps = 0.f, ps2 = 0.f, p[kDecUnroll];
#pragma unroll
        for (int u = 0; u < kDecUnroll; ++u) {
          p[u] = ok[u] ? __expf(a[u][g] - mx) : 0.f;
          ps += p[u]; ps2 = fmaf(p[u], p[u], ps2);
        }
        L[g] = fmaf(L[g], alpha, ps);
        Q2[g] = fmaf(Q2[g], alpha * alpha, ps2);
        m[g] = mx;
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          float t = acc[g][e] * alpha;
#pragma unroll
          for (int u = 0; u < kDecUnroll; ++u) if (ok[u]) t = fmaf(p[u], vf[u][e], t);
          acc[g][e] = t;
        }
      }
    }
  }

  // ---- merge the lane groups of the CTA ------------------------------------------------------
  __shared__ float s_m[kDecWarps * 8][GMAX];           // up to 8 groups per warp (DK = 32)
  __shared__ float s_acc[kDecWarps][GMAX][DK];
  __shared__ float s_l[kDecWarps][GMAX], s_q2[kDecWarps][GMAX];
  if (sub == 0) {
#pragma unroll
    for (int g = 0; g < GMAX; ++g) if (g < G) s_m[warp * GPW + grp][g] = m[g];
  }
  __syncthreads();
#pragma unroll
  for (int g = 0; g < GMAX; ++g) {
    if (g < G) {
      float M = kNegBig;
      for (int i = 0; i < kDecWarps * GPW; ++i) M = fmaxf(M, s_m[i][g]);
      const float w = __expf(m[g] - M);
      float l = L[g] * w, q2 = Q2[g] * w * w;
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[g][e] *= w;
      // sum over the GPW groups of this warp
#pragma unroll
      for (int o = LPR; o < 32; o <<= 1) {
        l += __shfl_xor_sync(0xffffffffu, l, o);
        q2 += __shfl_xor_sync(0xffffffffu, q2, o);
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[g][e] += __shfl_xor_sync(0xffffffffu, acc[g][e], o);
      }
      if (grp == 0) {
#pragma unroll
        for (int e = 0; e < 8; ++e) s_acc[warp][g][d0 + e] = acc[g][e];
        if (sub == 0) { s_l[warp][g] = l; s_q2[warp][g] = q2; }
      }
      m[g] = M;
    }
  }
  __syncthreads();
  for (int i = tid; i < G * DK; i += blockDim.x) {
    const int g = i / DK, d = i - g * DK;
    float s = 0.f;
#pragma unroll
    for (int w = 0; w < kDecWarps; ++w) s += s_acc[w][g][d];
    const int64_t bh = (int64_t)b * H + kvh * G + g;
    sacc[(bh * n_splits + split) * DK + d] = s;
  }
  if (tid < G) {
    const int g = tid;
    float l = 0.f, q2 = 0.f, M = kNegBig;
    for (int w = 0; w < kDecWarps; ++w) { l += s_l[w][g]; q2 += s_q2[w][g]; }
    for (int i = 0; i < kDecWarps * GPW; ++i) M = fmaxf(M, s_m[i][g]);
    const int64_t bh = (int64_t)b * H + kvh * G + g;
    *reinterpret_cast<float4*>(stats + dec_stats_off(bh, split, n_splits)) = make_float4(M, l, q2, 0.f);
  }
}

// Merge the key-range partials of one (sequence, head), fold the null sink, emit c and mag.
template <typename T>
__global__ void polar_decode_merge_kernel(const float* __restrict__ scratch,
                                          const int32_t* __restrict__ context_lens,
                                          const float* __restrict__ v_null,
                                          const float* __restrict__ spg,
                                          const float* __restrict__ null_base,
                                          const float* __restrict__ sps,
                                          const float* __restrict__ beta, T* __restrict__ c,
                                          T* __restrict__ mag, int B, int H, int dk, int n_splits,
                                          int window, int max_ctx, float eps, const T* __restrict__ gate,
                                          int64_t gate_sb, int64_t gate_sh, int64_t c_sb, int64_t mag_sb) {
  const int bh = blockIdx.x, b = bh / H, h = bh % H;
  const int tid = threadIdx.x;
  const float* stats = scratch + (int64_t)bh * n_splits * 4;
  const float* sacc = scratch + (int64_t)B * H * n_splits * 4 + (int64_t)bh * n_splits * dk;
  __shared__ float s_red[32];
  __shared__ float s_bc;
  // The weights e^(m_i - M) of the partials are worked out once, by the first warp, from one round of independent
  // 16-byte loads, and kept in shared memory; every thread then sums its channels over the partials with loads
  // that do not depend on one another.  (More than kMergeStaged partials: the plain loops.)
  constexpr int kMergeStaged = 128;
  __shared__ float s_w[kMergeStaged];
  __shared__ float s_mlq[3];
  const bool staged = n_splits <= kMergeStaged;
  float M = kNegBig, L = 0.f, Q2 = 0.f;
  if (staged) {
    if (tid < 32) {
      float4 st[kMergeStaged / 32];
      float m = kNegBig;
#pragma unroll
      for (int i = 0; i < kMergeStaged / 32; ++i) {
        const int sp = tid + 32 * i;
        st[i] = sp < n_splits ? *reinterpret_cast<const float4*>(stats + sp * 4) : make_float4(kNegBig, 0.f, 0.f, 0.f);
        m = fmaxf(m, st[i].x);
      }
      m = warp_max(m);
      float l = 0.f, q2 = 0.f;
#pragma unroll
      for (int i = 0; i < kMergeStaged / 32; ++i) {
        const int sp = tid + 32 * i;
        const float w = __expf(st[i].x - m);
        if (sp < n_splits) s_w[sp] = w;
        l = fmaf(st[i].y, w, l);
        q2 = fmaf(st[i].z, w * w, q2);
      }
      l = warp_sum(l); q2 = warp_sum(q2);
      if (tid == 0) { s_mlq[0] = m; s_mlq[1] = l; s_mlq[2] = q2; }
    }
    __syncthreads();
    M = s_mlq[0]; L = s_mlq[1]; Q2 = s_mlq[2];
  } else {
    for (int sp = 0; sp < n_splits; ++sp) M = fmaxf(M, stats[sp * 4]);
    for (int sp = 0; sp < n_splits; ++sp) {
      const float w = __expf(stats[sp * 4] - M);
      L = fmaf(stats[sp * 4 + 1], w, L);
      Q2 = fmaf(stats[sp * 4 + 2], w * w, Q2);
    }
  }
  int n = context_lens[b];
  n = max(0, min(n, max_ctx));
  const float nf = fmaxf(window > 0 ? fminf((float)n, (float)window) : (float)n, 1.0f);
  const float temp = 1.0f + spg[h] * logf(nf);
  const float a_n = temp * (null_base[h] + sps[h] * sqrtf(logf(nf + 1.0f)));
  const float Mn = fmaxf(M, a_n);
  const float al = __expf(M - Mn);
  const float p_n = __expf(a_n - Mn);
  L *= al; Q2 *= al * al;
  const float Z = L + p_n;

  float sq = 0.f;
  float sv[4];                                            // dk <= 4 * blockDim.x
  int cnt = 0;
  for (int d = tid; d < dk; d += blockDim.x, ++cnt) {
    float s = 0.f;
    if (staged) {
      int sp = 0;
      for (; sp + 8 <= n_splits; sp += 8) {               // eight independent loads in flight
        float x[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) x[u] = sacc[(sp + u) * dk + d];
#pragma unroll
        for (int u = 0; u < 8; ++u) s = fmaf(x[u], s_w[sp + u], s);
      }
      for (; sp < n_splits; ++sp) s = fmaf(sacc[sp * dk + d], s_w[sp], s);
    } else {
      for (int sp = 0; sp < n_splits; ++sp) s = fmaf(sacc[sp * dk + d], __expf(stats[sp * 4] - M), s);
    }
    s = s * al + p_n * v_null[h * dk + d];
    sv[cnt] = s; sq = fmaf(s, s, sq);
  }
  sq = warp_sum(sq);
  if ((tid & 31) == 0) s_red[tid >> 5] = sq;
  __syncthreads();
  if (tid == 0) {
    float t = 0.f;
    for (int w = 0; w < (blockDim.x + 31) / 32; ++w) t += s_red[w];
    s_bc = 1.0f / fmaxf(sqrtf(t), eps);
  }
  __syncthreads();
  const float inv = s_bc;
  cnt = 0;
  T* crow = c + (c_sb ? (int64_t)b * c_sb + (int64_t)h * dk : (int64_t)bh * dk);
  for (int d = tid; d < dk; d += blockDim.x, ++cnt) {
    float o = sv[cnt] * inv;
    if (gate != nullptr)                                   // c * sigmoid(gate), rounded where the separate ops round
      o = round_through<T>(o) * round_through<T>(1.0f / (1.0f + __expf(-to_f32(gate[b * gate_sb + h * gate_sh + d]))));
    crow[d] = from_f32<T>(o);
  }
  if (tid == 0) {
    const float n_eff = L * L / fmaxf(Q2, 1e-30f);
    const float m_eff = n_eff * (L / fmaxf(Z, eps));
    mag[mag_sb ? (int64_t)b * mag_sb + h : (int64_t)bh] = from_f32<T>(tanhf(beta[h] * log1pf(m_eff)));
  }
}

// tensor-core split kernel for 16-bit caches (polar_decode_mma.cu)
bool polar_decode_mma_supported(const atma_polar_decode_args& a);
bool polar_decode_mma_appends(const atma_polar_decode_args& a);
int polar_decode_split_mma(const atma_polar_decode_args& a, cudaStream_t st);

template <typename T>
int launch_decode(const atma_polar_decode_args& a, cudaStream_t st) {
  dim3 grid(a.n_splits, a.Hkv, a.B), block(kDecWarps * 32);
  const int G = a.H / a.Hkv;
  if (polar_decode_mma_supported(a)) {
    int rc = polar_decode_split_mma(a, st);
    if (rc != ATMA_OK || a.skip_merge) return rc;
    polar_decode_merge_kernel<T><<<a.B * a.H, 128, 0, st>>>(
        a.scratch, a.context_lens, a.v_null, a.spg, a.null_base, a.sps, a.beta, (T*)a.c, (T*)a.mag,
        a.B, a.H, a.dk, a.n_splits, a.window, a.max_blocks * a.block_size, a.eps, (const T*)a.gate, a.gate_sb, a.gate_sh,
        a.c_sb, a.mag_sb);
    return launch_status("polar_decode (merge)");
  }
#define ATMA_LAUNCH(DKK, GM)                                                                    \
  polar_decode_split_kernel<T, DKK, GM><<<grid, block, 0, st>>>(                                \
      (const T*)a.q, (const T*)a.k_cache, (const T*)a.v_cache, a.block_tables, a.bt_stride,     \
      a.context_lens, a.temp_lens, a.spg, a.scratch, a.B, a.H, a.Hkv, a.block_size, a.max_blocks,            \
      a.num_blocks, a.n_splits, a.window)
#define ATMA_CASE(DKK)                                                                          \
  case DKK:                                                                                     \
    if (G <= 1) ATMA_LAUNCH(DKK, 1); else if (G <= 2) ATMA_LAUNCH(DKK, 2);                      \
    else if (G <= 4) ATMA_LAUNCH(DKK, 4); else ATMA_LAUNCH(DKK, 8);                             \
    break;
  switch (a.dk) {
    ATMA_CASE(32) ATMA_CASE(64) ATMA_CASE(128) ATMA_CASE(256)
    default: return fail(ATMA_ERR_UNSUPPORTED, "polar_decode: head_dim %d not in {32,64,128,256}", a.dk);
  }
#undef ATMA_CASE
#undef ATMA_LAUNCH
  int rc = launch_status("polar_decode (split)");
  if (rc != ATMA_OK || a.skip_merge) return rc;
  polar_decode_merge_kernel<T><<<a.B * a.H, 128, 0, st>>>(
      a.scratch, a.context_lens, a.v_null, a.spg, a.null_base, a.sps, a.beta, (T*)a.c, (T*)a.mag,
      a.B, a.H, a.dk, a.n_splits, a.window, a.max_blocks * a.block_size, a.eps, (const T*)a.gate, a.gate_sb, a.gate_sh,
      a.c_sb, a.mag_sb);
  return launch_status("polar_decode (merge)");
}

}  // namespace atma

using namespace atma;

extern "C" int64_t atma_polar_decode_scratch_floats(int B, int H, int dk, int n_splits) {
  return (int64_t)B * H * n_splits * (4 + dk);
}

extern "C" int atma_polar_decode_appends(const atma_polar_decode_args* args) {
  return (args != nullptr && atma::polar_decode_mma_appends(*args)) ? 1 : 0;
}

extern "C" int atma_polar_decode(const atma_polar_decode_args* args, void* stream) {
  ATMA_REQUIRE(args != nullptr, "polar_decode: null args");
  const atma_polar_decode_args& a = *args;
  ATMA_REQUIRE(dtype_ok(a.dtype), "polar_decode: unsupported dtype %d", a.dtype);
  ATMA_REQUIRE(a.Hkv > 0 && a.H % a.Hkv == 0, "polar_decode: H=%d not a multiple of Hkv=%d", a.H, a.Hkv);
  ATMA_REQUIRE(a.H / a.Hkv <= kDecMaxG || polar_decode_mma_supported(a),
               "polar_decode: GQA group size %d > %d", a.H / a.Hkv, kDecMaxG);
  ATMA_REQUIRE(a.n_splits >= 1 && a.n_splits <= 1024, "polar_decode: n_splits=%d", a.n_splits);
  ATMA_REQUIRE(a.block_size > 0 && a.max_blocks > 0 && a.num_blocks > 0, "polar_decode: empty cache geometry");
  ATMA_REQUIRE(a.scratch != nullptr, "polar_decode: scratch is required");
  ATMA_REQUIRE((uintptr_t)a.q % 16 == 0 && (uintptr_t)a.k_cache % 16 == 0 && (uintptr_t)a.v_cache % 16 == 0 &&
                   (uintptr_t)a.scratch % 16 == 0,
               "polar_decode: q / caches / scratch must be 16-byte aligned");
  if (a.B <= 0) return ATMA_OK;
  int rc = ATMA_OK;
  ATMA_DISPATCH_DTYPE(a.dtype, T, { rc = launch_decode<T>(a, (cudaStream_t)stream); });
  return rc;
}

extern "C" int atma_polar_decode_merge(const atma_polar_decode_args* args, void* stream) {
  ATMA_REQUIRE(args != nullptr, "polar_decode_merge: null args");
  const atma_polar_decode_args& a = *args;
  ATMA_REQUIRE(dtype_ok(a.dtype), "polar_decode_merge: unsupported dtype %d", a.dtype);
  ATMA_REQUIRE(a.n_splits >= 1 && a.n_splits <= 4096, "polar_decode_merge: n_splits=%d", a.n_splits);
  ATMA_REQUIRE(a.scratch != nullptr && a.context_lens != nullptr && a.c != nullptr && a.mag != nullptr, "polar_decode_merge: missing buffers");
  ATMA_REQUIRE(a.dk >= 1 && a.dk <= 256, "polar_decode_merge: head_dim %d", a.dk);
  if (a.B <= 0) return ATMA_OK;
  ATMA_DISPATCH_DTYPE(a.dtype, T, {
    polar_decode_merge_kernel<T><<<a.B * a.H, 128, 0, (cudaStream_t)stream>>>(
        a.scratch, a.context_lens, a.v_null, a.spg, a.null_base, a.sps, a.beta, (T*)a.c, (T*)a.mag, a.B, a.H, a.dk, a.n_splits,
        a.window, 0x7fffffff, a.eps, (const T*)a.gate, a.gate_sb, a.gate_sh, a.c_sb, a.mag_sb);
  });
  return launch_status("polar_decode (merge)");
}

// ---- decode without caller scratch ---------------------------------------------------------
// Some hosts of this library may not allocate device memory at the point where they decode:
// an inference engine that sizes its KV cache to fill the GPU and hands every remaining byte
// to the cache has nothing left to ask cudaMalloc for, and a serving loop that runs inside a
// pre-planned memory arena is not allowed to.  For them the split partials live in a
// fixed-size array that is part of the library image; every GPU that loads the library holds
// these 4 MiB until the process exits.
constexpr int64_t kStaticScratchFloats = 1 << 20;            // 4 MiB
static __device__ __align__(256) float g_decode_scratch[kStaticScratchFloats];

namespace {
constexpr int kMaxDevices = 64;
float* g_scratch_ptr[kMaxDevices] = {nullptr};               // device address of the array, per GPU
}  // namespace

extern "C" int64_t atma_polar_decode_static_max_floats(void) { return kStaticScratchFloats; }

extern "C" int atma_polar_decode_static(const atma_polar_decode_args* args, void* stream) {
  ATMA_REQUIRE(args != nullptr, "polar_decode_static: null args");
  const int64_t need = atma_polar_decode_scratch_floats(args->B, args->H, args->dk, args->n_splits);
  ATMA_REQUIRE(args->B >= 0 && args->H > 0 && args->dk > 0 && args->n_splits >= 1,
               "polar_decode_static: bad shape");
  ATMA_REQUIRE(need <= kStaticScratchFloats,
               "polar_decode_static: B*H*n_splits*(4+dk) = %lld floats exceeds the built-in scratch of "
               "%lld floats; lower n_splits or the batch, or call atma_polar_decode with caller scratch",
               (long long)need, (long long)kStaticScratchFloats);
  int dev = 0;
  ATMA_CUDA_OK(cudaGetDevice(&dev));
  ATMA_REQUIRE(dev >= 0 && dev < kMaxDevices, "polar_decode_static: device ordinal %d out of range", dev);
  if (g_scratch_ptr[dev] == nullptr) {
    // In host code the array's name is only a handle for the runtime; the address a kernel can
    // use has to be asked for, once per device, with that device current.
    float* p = nullptr;
    ATMA_CUDA_OK(cudaGetSymbolAddress((void**)&p, g_decode_scratch));
    ATMA_REQUIRE(p != nullptr, "polar_decode_static: no device address for the built-in scratch");
    g_scratch_ptr[dev] = p;
  }
  atma_polar_decode_args a = *args;
  a.scratch = g_scratch_ptr[dev];
  return atma_polar_decode(&a, stream);
}
