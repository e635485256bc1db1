// Gated-delta decode step: one token per sequence, state [dk][dv] fp32 read and written
// once, in place, through a slot table.
//
//   Sd = gamma * S;  pred_v = sum_k kn_k Sd[k,v];  u_v = beta (v_v - pred_v)
//   S' = Sd + kn u^T (stored);  r_v = sum_k qn_k S'[k,v]
//
// One CTA owns a [dk] x [32] column slice of one (sequence, head) state, held entirely in
// registers between the read and the write: 8 lanes x float4 span the 32 columns, the
// other 4 lane groups x NWARPS warps stride the dk rows, so every warp-level access is
// four full 128-byte rows.  HBM traffic is exactly one read and one write of the state.
#include "common.cuh"

namespace atma {

constexpr int kStepCols = 32;     // state columns per CTA
constexpr int kStepWarps = 4;
constexpr int kStepMaxRowsPerThread = 16;   // dk <= 16 * 4 * kStepWarps = 256

template <typename T>
__global__ void __launch_bounds__(kStepWarps * 32)
gated_delta_step_kernel(const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v,
                        int64_t q_sb, int64_t q_sh, int64_t k_sb, int64_t k_sh, int64_t v_sb,
                        int64_t v_sh, const float* __restrict__ gamma,
                        const float* __restrict__ beta, float* __restrict__ state, int64_t state_ss,
                        int64_t state_sh, const int64_t* __restrict__ slots, float* __restrict__ r,
                        int H, int dk, int dv, float eps) {
  const int bh = blockIdx.x;
  const int b = bh / H, h = bh % H;
  const int col0 = blockIdx.y * kStepCols;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int cg = lane & 7;          // float4 column group inside the slice
  const int rg = (lane >> 3) + 4 * warp;   // row group: rows rg, rg + 4*NW, ...
  constexpr int RSTRIDE = 4 * kStepWarps;

  __shared__ float s_q[256], s_k[256];
  __shared__ float s_red[kStepWarps][kStepCols];
  __shared__ float s_norm[2];

  const int64_t slot = slots[b];
  const int col = col0 + cg * 4;
  const bool col_ok = col < dv;     // dv % 4 == 0 is required by the host wrapper
  if (slot < 0) {                   // padded batch row: no state, defined output
    if (tid < kStepCols && col0 + tid < dv) r[((int64_t)b * H + h) * dv + col0 + tid] = 0.f;
    return;
  }

  // the state slice first: its loads are in flight while q and k are normalised
  float* sp = state + slot * state_ss + h * state_sh;
  float4 S[kStepMaxRowsPerThread];
#pragma unroll
  for (int i = 0; i < kStepMaxRowsPerThread; ++i) {
    const int row = rg + i * RSTRIDE;
    S[i] = (row < dk && col_ok) ? *reinterpret_cast<const float4*>(sp + (int64_t)row * dv + col)
                                : make_float4(0.f, 0.f, 0.f, 0.f);
  }

  // q, k -> shared, with their L2 norms (F.normalize: x / max(||x||, eps))
  float qs = 0.f, ks = 0.f;
  for (int i = tid; i < dk; i += blockDim.x) {
    float qv = to_f32(q[b * q_sb + h * q_sh + i]);
    float kv = to_f32(k[b * k_sb + h * k_sh + i]);
    s_q[i] = qv; s_k[i] = kv;
    qs += qv * qv; ks += kv * kv;
  }
  qs = warp_sum(qs); ks = warp_sum(ks);
  if (lane == 0) { s_red[warp][0] = qs; s_red[warp][1] = ks; }
  __syncthreads();
  if (tid == 0) {
    float a = 0.f, c = 0.f;
    for (int w = 0; w < kStepWarps; ++w) { a += s_red[w][0]; c += s_red[w][1]; }
    s_norm[0] = 1.f / fmaxf(sqrtf(a), eps);
    s_norm[1] = 1.f / fmaxf(sqrtf(c), eps);
  }
  __syncthreads();
  const float qinv = s_norm[0], kinv = s_norm[1];
  const float gm = gamma[b * H + h], bt = beta[b * H + h];

  float4 pred = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
  for (int i = 0; i < kStepMaxRowsPerThread; ++i) {
    const int row = rg + i * RSTRIDE;
    if (row < dk && col_ok) {
      float4 s = S[i];
      s.x *= gm; s.y *= gm; s.z *= gm; s.w *= gm;
      const float kn = s_k[row] * kinv;
      pred.x = fmaf(kn, s.x, pred.x); pred.y = fmaf(kn, s.y, pred.y);
      pred.z = fmaf(kn, s.z, pred.z); pred.w = fmaf(kn, s.w, pred.w);
      S[i] = s;
    } else {
      S[i] = make_float4(0.f, 0.f, 0.f, 0.f);
    }
  }
  // reduce pred over the 4 row groups of the warp (lane bits 3,4), then over warps
#pragma unroll
  for (int o = 8; o <= 16; o <<= 1) {
    pred.x += __shfl_xor_sync(0xffffffffu, pred.x, o); pred.y += __shfl_xor_sync(0xffffffffu, pred.y, o);
    pred.z += __shfl_xor_sync(0xffffffffu, pred.z, o); pred.w += __shfl_xor_sync(0xffffffffu, pred.w, o);
  }
  __syncthreads();                  // s_red reuse
  if (lane < 8) *reinterpret_cast<float4*>(&s_red[warp][cg * 4]) = pred;
  __syncthreads();
  float4 u = make_float4(0.f, 0.f, 0.f, 0.f);
  if (col_ok) {
    float4 p = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int w = 0; w < kStepWarps; ++w) {
      float4 t = *reinterpret_cast<const float4*>(&s_red[w][cg * 4]);
      p.x += t.x; p.y += t.y; p.z += t.z; p.w += t.w;
    }
    const T* vp = v + b * v_sb + h * v_sh + col;
    u.x = bt * (to_f32(vp[0]) - p.x); u.y = bt * (to_f32(vp[1]) - p.y);
    u.z = bt * (to_f32(vp[2]) - p.z); u.w = bt * (to_f32(vp[3]) - p.w);
  }
  float4 rd = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
  for (int i = 0; i < kStepMaxRowsPerThread; ++i) {
    const int row = rg + i * RSTRIDE;
    if (row < dk && col_ok) {
      const float kn = s_k[row] * kinv, qn = s_q[row] * qinv;
      float4 s = S[i];
      s.x = fmaf(kn, u.x, s.x); s.y = fmaf(kn, u.y, s.y); s.z = fmaf(kn, u.z, s.z); s.w = fmaf(kn, u.w, s.w);
      *reinterpret_cast<float4*>(sp + (int64_t)row * dv + col) = s;
      rd.x = fmaf(qn, s.x, rd.x); rd.y = fmaf(qn, s.y, rd.y); rd.z = fmaf(qn, s.z, rd.z); rd.w = fmaf(qn, s.w, rd.w);
    }
  }
#pragma unroll
  for (int o = 8; o <= 16; o <<= 1) {
    rd.x += __shfl_xor_sync(0xffffffffu, rd.x, o); rd.y += __shfl_xor_sync(0xffffffffu, rd.y, o);
    rd.z += __shfl_xor_sync(0xffffffffu, rd.z, o); rd.w += __shfl_xor_sync(0xffffffffu, rd.w, o);
  }
  __syncthreads();
  if (lane < 8) *reinterpret_cast<float4*>(&s_red[warp][cg * 4]) = rd;
  __syncthreads();
  if (tid < 8 && col0 + tid * 4 < dv) {
    float4 o = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int w = 0; w < kStepWarps; ++w) {
      float4 t = *reinterpret_cast<const float4*>(&s_red[w][tid * 4]);
      o.x += t.x; o.y += t.y; o.z += t.z; o.w += t.w;
    }
    *reinterpret_cast<float4*>(r + ((int64_t)b * H + h) * dv + col0 + tid * 4) = o;
  }
}

// ---- the same step with its surroundings folded in (dk = dv = 128) ----------------------------------
// One CTA of 256 threads owns the whole [128][128] state of one (sequence, head): thread (cg = t & 31,
// rg = t >> 5) holds the float4 column group cg of rows rg, rg + 8, ... - sixteen 16-byte loads in
// flight per thread, every warp access one full 512-byte state row.  k and v are read from their
// un-expanded KV head, gamma and beta may come as the logits of their projections, and the read-out
// can leave as RMSNorm(r) * sigmoid(gate) in the activation dtype (the operand of mem.proj).
struct StepWideArgs {
  const void *q, *k, *v;
  int64_t q_sb, q_sh, k_sb, k_sh, v_sb, v_sh;
  const float *gamma, *beta;
  const void *g_logit, *b_logit; int64_t logit_sb; float gamma_bias, beta_bias;
  float* state; int64_t state_ss, state_sh;
  const int64_t* slots;
  float* r;
  const void* gate; int64_t gate_sb; void* out; int64_t out_sb;
  int H, G; float eps, rms_eps;
};

template <typename T>
__global__ void __launch_bounds__(256, 2)
gated_delta_step_wide_kernel(const StepWideArgs a) {
  constexpr int D = 128, NW = 8, RPT = 16;
  const int bh = blockIdx.x, b = bh / a.H, h = bh % a.H, hk = h / a.G;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  __shared__ float s_q[D], s_k[D];
  __shared__ __align__(16) float s_red[NW][D];
  __shared__ float s_part[2][NW];

  const int64_t slot = a.slots[b];
  if (slot < 0) {                                       // padded batch row: no state, defined output
    if (tid < D) {
      if (a.out != nullptr) static_cast<T*>(a.out)[b * a.out_sb + h * D + tid] = from_f32<T>(0.f);
      else a.r[((int64_t)b * a.H + h) * D + tid] = 0.f;
    }
    return;
  }
  float* sp = a.state + slot * a.state_ss + h * a.state_sh + lane * 4;
  float4 S[RPT];
#pragma unroll
  for (int i = 0; i < RPT; ++i) S[i] = *reinterpret_cast<const float4*>(sp + (int64_t)(warp + NW * i) * D);

  float qs = 0.f, ks = 0.f;
  if (tid < D) {
    const float qv = to_f32(static_cast<const T*>(a.q)[b * a.q_sb + h * a.q_sh + tid]);
    const float kv = to_f32(static_cast<const T*>(a.k)[b * a.k_sb + hk * a.k_sh + tid]);
    s_q[tid] = qv; s_k[tid] = kv;
    qs = qv * qv; ks = kv * kv;
  }
  qs = warp_sum(qs); ks = warp_sum(ks);
  if (lane == 0) { s_part[0][warp] = qs; s_part[1][warp] = ks; }
  float gm, bt;
  if (a.g_logit != nullptr) {
    gm = 1.0f / (1.0f + __expf(-(to_f32(static_cast<const T*>(a.g_logit)[b * a.logit_sb + h]) + a.gamma_bias)));
    bt = 1.0f / (1.0f + __expf(-(to_f32(static_cast<const T*>(a.b_logit)[b * a.logit_sb + h]) + a.beta_bias)));
  } else {
    gm = a.gamma[b * a.H + h]; bt = a.beta[b * a.H + h];
  }
  __syncthreads();
  float qn2 = 0.f, kn2 = 0.f;
#pragma unroll
  for (int w = 0; w < 4; ++w) { qn2 += s_part[0][w]; kn2 += s_part[1][w]; }   // the 128 channels sit in warps 0-3
  const float qinv = 1.f / fmaxf(sqrtf(qn2), a.eps), kinv = 1.f / fmaxf(sqrtf(kn2), a.eps);

  float4 pred = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
  for (int i = 0; i < RPT; ++i) {
    float4 s = S[i];
    s.x *= gm; s.y *= gm; s.z *= gm; s.w *= gm;
    const float kn = s_k[warp + NW * i] * kinv;
    pred.x = fmaf(kn, s.x, pred.x); pred.y = fmaf(kn, s.y, pred.y);
    pred.z = fmaf(kn, s.z, pred.z); pred.w = fmaf(kn, s.w, pred.w);
    S[i] = s;
  }
  *reinterpret_cast<float4*>(&s_red[warp][lane * 4]) = pred;
  __syncthreads();
  float4 u;
  {
    float4 p = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int w = 0; w < NW; ++w) {
      const float4 t = *reinterpret_cast<const float4*>(&s_red[w][lane * 4]);
      p.x += t.x; p.y += t.y; p.z += t.z; p.w += t.w;
    }
    const T* vp = static_cast<const T*>(a.v) + b * a.v_sb + hk * a.v_sh + lane * 4;
    u.x = bt * (to_f32(vp[0]) - p.x); u.y = bt * (to_f32(vp[1]) - p.y);
    u.z = bt * (to_f32(vp[2]) - p.z); u.w = bt * (to_f32(vp[3]) - p.w);
  }
  __syncthreads();                                      // s_red is reused below
  float4 rd = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
  for (int i = 0; i < RPT; ++i) {
    const int row = warp + NW * i;
    const float kn = s_k[row] * kinv, qn = s_q[row] * qinv;
    float4 s = S[i];
    s.x = fmaf(kn, u.x, s.x); s.y = fmaf(kn, u.y, s.y); s.z = fmaf(kn, u.z, s.z); s.w = fmaf(kn, u.w, s.w);
    *reinterpret_cast<float4*>(sp + (int64_t)row * D) = s;
    rd.x = fmaf(qn, s.x, rd.x); rd.y = fmaf(qn, s.y, rd.y); rd.z = fmaf(qn, s.z, rd.z); rd.w = fmaf(qn, s.w, rd.w);
  }
  *reinterpret_cast<float4*>(&s_red[warp][lane * 4]) = rd;
  __syncthreads();
  float rv = 0.f;
  if (tid < D) {
#pragma unroll
    for (int w = 0; w < NW; ++w) rv += s_red[w][tid];
    if (a.out == nullptr) { a.r[((int64_t)b * a.H + h) * D + tid] = rv; return; }
  }
  if (a.out == nullptr) return;
  float ss = tid < D ? rv * rv : 0.f;                  // RMSNorm(r) * sigmoid(gate)
  ss = warp_sum(ss);
  if (lane == 0) s_part[0][warp] = ss;
  __syncthreads();
  if (tid < D) {
    const float tot = s_part[0][0] + s_part[0][1] + s_part[0][2] + s_part[0][3];
    const float rs = rsqrtf(tot / (float)D + a.rms_eps);
    const float g = to_f32(static_cast<const T*>(a.gate)[b * a.gate_sb + h * D + tid]);
    static_cast<T*>(a.out)[b * a.out_sb + h * D + tid] =
        from_f32<T>(round_through<T>(rv * rs) * round_through<T>(1.0f / (1.0f + __expf(-g))));
  }
}

}  // namespace atma

using namespace atma;

extern "C" int atma_gated_delta_decode_step_fused(const void* q, const void* k, const void* v,
                                                  int64_t q_sb, int64_t q_sh, int64_t k_sb, int64_t k_sh,
                                                  int64_t v_sb, int64_t v_sh, int dtype, int Hkv,
                                                  const float* gamma, const float* beta,
                                                  const void* g_logit, const void* b_logit, int64_t logit_sb,
                                                  float gamma_bias, float beta_bias,
                                                  float* state, int64_t state_ss, int64_t state_sh,
                                                  const int64_t* slots, float* r,
                                                  const void* gate, int64_t gate_sb, void* out, int64_t out_sb,
                                                  int B, int H, int dk, int dv, float eps, float rms_eps, void* stream) {
  ATMA_REQUIRE(dtype_ok(dtype), "gated_delta_decode_step_fused: unsupported dtype %d", dtype);
  ATMA_REQUIRE(dk == 128 && dv == 128, "gated_delta_decode_step_fused: needs dk = dv = 128 (got %d, %d)", dk, dv);
  ATMA_REQUIRE(Hkv > 0 && H % Hkv == 0, "gated_delta_decode_step_fused: H=%d is not a multiple of Hkv=%d", H, Hkv);
  ATMA_REQUIRE((gamma != nullptr && beta != nullptr) || (g_logit != nullptr && b_logit != nullptr),
               "gated_delta_decode_step_fused: pass gamma and beta, or their two logit tensors");
  ATMA_REQUIRE((gate != nullptr) == (out != nullptr) && (out != nullptr || r != nullptr),
               "gated_delta_decode_step_fused: pass gate and out together, or r");
  ATMA_REQUIRE(((uintptr_t)state % 16 == 0) && (state_ss % 4 == 0) && (state_sh % 4 == 0),
               "gated_delta_decode_step_fused: the state rows must be 16-byte aligned");
  if (B <= 0 || H <= 0) return ATMA_OK;
  StepWideArgs a{q, k, v, q_sb, q_sh, k_sb, k_sh, v_sb, v_sh, gamma, beta, g_logit, b_logit, logit_sb, gamma_bias, beta_bias,
                 state, state_ss, state_sh, slots, r, gate, gate_sb, out, out_sb, H, H / Hkv, eps, rms_eps};
  ATMA_DISPATCH_DTYPE(dtype, T, {
    gated_delta_step_wide_kernel<T><<<B * H, 256, 0, (cudaStream_t)stream>>>(a);
  });
  return launch_status("gated_delta_decode_step_fused");
}

extern "C" int atma_gated_delta_decode_step(const void* q, const void* k, const void* v,
                                            int64_t q_sb, int64_t q_sh, int64_t k_sb, int64_t k_sh,
                                            int64_t v_sb, int64_t v_sh, int dtype,
                                            const float* gamma, const float* beta, float* state,
                                            int64_t state_ss, int64_t state_sh,
                                            const int64_t* slots, float* r, int B, int H, int dk,
                                            int dv, float eps, void* stream) {
  ATMA_REQUIRE(dtype_ok(dtype), "gated_delta_decode_step: unsupported dtype %d", dtype);
  ATMA_REQUIRE(dk >= 1 && dk <= 256, "gated_delta_decode_step: dk=%d outside 1..256", dk);
  ATMA_REQUIRE(dv >= 4 && dv % 4 == 0, "gated_delta_decode_step: dv=%d must be a multiple of 4", dv);
  ATMA_REQUIRE(((uintptr_t)state % 16 == 0) && (state_ss % 4 == 0) && (state_sh % 4 == 0) &&
                   ((uintptr_t)r % 16 == 0),
               "gated_delta_decode_step: state / r must be 16-byte aligned");
  if (B <= 0 || H <= 0) return ATMA_OK;
  dim3 grid(B * H, (dv + kStepCols - 1) / kStepCols), block(kStepWarps * 32);
  ATMA_DISPATCH_DTYPE(dtype, T, {
    gated_delta_step_kernel<T><<<grid, block, 0, (cudaStream_t)stream>>>(
        (const T*)q, (const T*)k, (const T*)v, q_sb, q_sh, k_sb, k_sh, v_sb, v_sh, gamma, beta,
        state, state_ss, state_sh, slots, r, H, dk, dv, eps);
  });
  return launch_status("gated_delta_decode_step");
}
