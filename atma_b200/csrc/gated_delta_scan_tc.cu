// Gated-delta chunked scan for 16-bit inputs, d_k = d_v = 128, chunk = 64: host side of the
// tensor-core path.
//
// Same factorisation as the fp32 kernel (gated_delta_scan.cu):
//   per chunk, independent of the state:  -W = -T diag(beta g) K,  U0 = T diag(beta) V,
//       Qg = diag(g) Q,  Kt = diag(g_C/g) K,  Rq = tril((g_p/g_s) q_p.k_s),  T = (I + A)^-1
//   per chunk, on the state S [dk][dv]:    U = U0 - W S;  O = Qg S + Rq U;  S <- g_C S + Kt^T U
// The chunk-local factors come from the tcgen05 kernel of gated_delta_local_sm100.cu (one record
// per chunk and head in scratch memory), the recurrence over the chunks from the tcgen05 kernel of
// gated_delta_scan_sm100.cu.  This file lays out the scratch, builds the packed-batch chunk
// offsets and sequences the two launches.
#include "common.cuh"
#include "gated_delta_scan.cuh"

namespace atma {

using namespace scan;

namespace {

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

// ---- one long sequence cut into segments (see gated_delta_scan_mma) -------------------------------
// Initial states of the first pass: per batch row, recurrence 0 walks segment 0 from the caller's
// initial state (or zero); for every later segment one recurrence starts from the identity (its
// final state is the segment's transfer matrix P) and one from zero (final state Q).
__global__ void seg_init_kernel(float* __restrict__ init, const float* __restrict__ user_init, int H, int per_row) {
  const int i = blockIdx.y, h = blockIdx.x;                    // recurrence, head
  const int b = i / per_row, j = i % per_row;
  float* dst = init + ((int64_t)i * H + h) * kD * kD;
  const float* src = (j == 0 && user_init != nullptr) ? user_init + ((int64_t)b * H + h) * kD * kD : nullptr;
  const bool ident = j > 0 && (j & 1) == 1;                     // j = 1, 3, 5 ...: the P recurrences
  for (int e = threadIdx.x; e < kD * kD; e += blockDim.x)
    dst[e] = src ? src[e] : ((ident && (e / kD) == (e % kD)) ? 1.f : 0.f);
}

// State at the start of every segment from the first pass's results: S_1 = end of segment 0,
// S_{s+1} = P_s S_s + Q_s; the last step gives the final state.  One CTA per (16 value columns,
// head, batch row); the columns of S are independent.
__global__ void __launch_bounds__(256)
seg_compose_kernel(const float* __restrict__ fin1, float* __restrict__ init2, float* __restrict__ final_state, int H, int NS) {
  __shared__ float Ss[kD][17];
  const int slab = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int per_row = 2 * NS - 1;
  const int k = threadIdx.x >> 1, c0 = (threadIdx.x & 1) * 8;
  auto plane = [&](const float* base, int rec) { return base + ((int64_t)rec * H + h) * kD * kD; };
  const float* s0 = plane(fin1, b * per_row);
  float acc[8];
#pragma unroll
  for (int c = 0; c < 8; ++c) acc[c] = s0[k * kD + 16 * slab + c0 + c];
  for (int s = 1; s <= NS; ++s) {
    if (s < NS) {
      float* dst = init2 + (((int64_t)b * (NS - 1) + (s - 1)) * H + h) * kD * kD;
#pragma unroll
      for (int c = 0; c < 8; ++c) dst[k * kD + 16 * slab + c0 + c] = acc[c];
    } else {
      if (final_state != nullptr) {
        float* dst = final_state + ((int64_t)b * H + h) * kD * kD;
#pragma unroll
        for (int c = 0; c < 8; ++c) dst[k * kD + 16 * slab + c0 + c] = acc[c];
      }
      break;
    }
    __syncthreads();
#pragma unroll
    for (int c = 0; c < 8; ++c) Ss[k][c0 + c] = acc[c];
    __syncthreads();
    const float* P = plane(fin1, b * per_row + 2 * s - 1) + k * kD;
    const float* Q = plane(fin1, b * per_row + 2 * s) + k * kD + 16 * slab + c0;
#pragma unroll
    for (int c = 0; c < 8; ++c) acc[c] = Q[c];
    // the row of P in four batches of eight independent 16-byte loads (the chain of segments is serial, so the
    // load latency of every step counts)
#pragma unroll 1
    for (int m0 = 0; m0 < kD; m0 += 32) {
      float4 pv[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) pv[u] = __ldg(reinterpret_cast<const float4*>(P + m0 + 4 * u));
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const float pm[4] = {pv[u].x, pv[u].y, pv[u].z, pv[u].w};
#pragma unroll
        for (int e = 0; e < 4; ++e)
#pragma unroll
          for (int c = 0; c < 8; ++c) acc[c] = fmaf(pm[e], Ss[m0 + 4 * u + e][c0 + c], acc[c]);
      }
    }
  }
}

}  // namespace

// Number of segments a sequence of NC chunks is cut into when the batch alone cannot fill the
// machine: the first pass runs 2 recurrences per later segment (transfer matrix and offset), so
// B * H * 2 * NS CTAs should fit the SM count; a segment should still be at least 32 chunks long.
int gated_delta_scan_segments(int B, int H, int NC, int requested) {
  const int sms = sm_count_of_current_device();
  int ns = requested > 0 ? requested : sms / (2 * B * H);
  if (ns > 16) ns = 16;
  if (ns > NC / 32) ns = NC / 32;
  while (ns >= 2 && B * (2 * ns - 1) > kMaxRec) --ns;
  return ns >= 2 ? ns : 1;
}

static int64_t seg_workspace_floats(int B, int H, int NS) {
  return NS < 2 ? 0 : (int64_t)B * H * kD * kD * (2 * (2 * NS - 1) + (NS - 1));
}

bool gated_delta_scan_mma_supported(int dtype, int dk, int dv) {
  return (dtype == ATMA_BF16 || dtype == ATMA_F16) && dk == kD && dv == kD;
}

static int64_t record_bytes(int B, int T, int H) {
  const int64_t NC = (T + kC - 1) / kC;
  return ((int64_t)B * H * NC * kRecBytes + 255) / 256 * 256 + ((int64_t)B * H * NC * sizeof(float) + 255) / 256 * 256;
}

// records | g_C | workspace of the segmented recurrence (sized for the largest segment count)
int64_t gated_delta_scan_mma_scratch_bytes(int B, int T, int H) {
  const int NC = (T + kC - 1) / kC;
  int64_t ws = 0;
  for (int ns = 2; ns <= 16; ++ns)
    if (gated_delta_scan_segments(B, H, NC, ns) == ns) ws = seg_workspace_floats(B, H, ns) * (int64_t)sizeof(float);
  return record_bytes(B, T, H) + ws + 256;
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
  return gated_delta_local_sm100(q, k, v, dtype == ATMA_BF16, g, beta, recs, gcs, B, T, H, Hkv, NC, normalize_qk, scale, VarLen{},
                                 (int64_t)B * T, st);
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
    map.state_row[i] = i;
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
  return record_bytes(1, (int)(NCu * kC), H) + (((int64_t)n_seqs + 1) * 4 + 255) / 256 * 256 + 256;
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
  int32_t* cu_chunks = reinterpret_cast<int32_t*>(recs + record_bytes(1, NCu * kC, H));
  varlen_chunk_offsets_kernel<<<1, 32, 0, st>>>(cu_seqlens, cu_chunks, n_seqs);
  VarLen var{cu_seqlens, cu_chunks, n_seqs, slots, has_initial, state_table, slot_stride, snapshots, snap_offsets, snap_chunks};
  const bool bf = dtype == ATMA_BF16;
  int rc = gated_delta_local_sm100(q, k, v, bf, g, beta, recs, gcs, 1, 0, H, Hkv, NCu, normalize_qk, scale, var, total_tokens, st);
  if (rc != ATMA_OK) return rc;
  return gated_delta_recur_sm100(recs, gcs, bf, (int64_t)H * NCu, initial_state, o, final_state, 0, H, NCu, n_seqs, RecMap{}, var,
                                 st);
}

// The whole scan.  `segments`: 1 = one recurrence per sequence; n > 1 = cut every sequence into n
// segments; 0 = choose (segments only when B * H CTAs would leave most of the machine idle).
// With segments the chunk axis is walked twice, both times with all segments side by side: a first
// pass yields each later segment's affine map S_out = P S_in + Q (segment 0 runs for real), a small
// kernel chains the maps into the state at the start of every segment, and a second pass runs the
// later segments from those states.  Latency drops by about n / 2 for about three times the
// recurrence work, so callers that run the scan beside other kernels ask for 1.
int gated_delta_scan_mma(const void* q, const void* k, const void* v, int dtype, const float* g, const float* beta,
                         const float* initial_state, void* o, float* final_state, void* scratch, int B, int T, int H,
                         int Hkv, int normalize_qk, float scale, int segments, cudaStream_t st) {
  int rc = gated_delta_scan_mma_factors(q, k, v, dtype, g, beta, scratch, B, T, H, Hkv, normalize_qk, scale, st);
  if (rc != ATMA_OK) return rc;
  const int NC = (T + kC - 1) / kC;
  const int NS = segments == 1 ? 1 : gated_delta_scan_segments(B, H, NC, segments);
  if (NS >= 2) {
    const uint8_t* recs = static_cast<const uint8_t*>(scratch);
    const float* gcs = gc_array(scratch, B, H, NC);
    float* ws = reinterpret_cast<float*>(static_cast<uint8_t*>(scratch) + record_bytes(B, T, H));
    const int per_row = 2 * NS - 1, n1 = B * per_row, n2 = B * (NS - 1);
    const int64_t plane = (int64_t)H * kD * kD;
    float* init1 = ws;
    float* fin1 = init1 + (int64_t)n1 * plane;
    float* init2 = fin1 + (int64_t)n1 * plane;
    const int seg = ((NC + NS - 1) / NS + 1) / 2 * 2;            // chunks per segment, even (the factor tiles pair chunks)
    seg_init_kernel<<<dim3(H, n1), 256, 0, st>>>(init1, initial_state, H, per_row);
    RecMap m1{}, m2{};
    for (int b = 0; b < B; ++b) {
      for (int j = 0; j < per_row; ++j) {
        const int i = b * per_row + j, s = (j + 1) / 2;            // j = 0: segment 0; then (P, Q) pairs
        m1.rec[i] = b; m1.o_row[i] = b;
        m1.zero_u0[i] = (j > 0 && (j & 1)) ? 1 : 0;
        m1.c_begin[i] = s * seg < NC ? s * seg : NC;
        m1.c_end[i] = (s + 1) * seg < NC ? (s + 1) * seg : NC;
        if (m1.c_end[i] <= m1.c_begin[i]) { m1.c_begin[i] = NC; m1.c_end[i] = NC; }
      }
      for (int s = 1; s < NS; ++s) {
        const int i = b * (NS - 1) + (s - 1);
        m2.rec[i] = b; m2.o_row[i] = b; m2.zero_u0[i] = 0;
        m2.c_begin[i] = s * seg < NC ? s * seg : NC;
        m2.c_end[i] = (s + 1) * seg < NC ? (s + 1) * seg : NC;
      }
    }
    const bool bf = dtype == ATMA_BF16;
    rc = launch_status("gated_delta_scan (segment setup)");
    if (rc != ATMA_OK) return rc;
    // pass 1 is one launch: the segment-0 recurrences write o, the (P, Q) recurrences carry state only
    // (o_row < 0); state_row keeps recurrence i on plane i of init1 / fin1
    for (int i = 0; i < n1; ++i) {
      m1.state_row[i] = i;
      if ((i % per_row) != 0) m1.o_row[i] = -1;
    }
    rc = gated_delta_recur_sm100(recs, gcs, bf, (int64_t)B * H * NC, init1, o, fin1, T, H, NC, n1, m1, VarLen{}, st);
    if (rc != ATMA_OK) return rc;
    seg_compose_kernel<<<dim3(kD / 16, H, B), 256, 0, st>>>(fin1, init2, final_state, H, NS);
    rc = launch_status("gated_delta_scan (segment states)");
    if (rc != ATMA_OK) return rc;
    for (int i = 0; i < n2; ++i) m2.state_row[i] = i;
    return gated_delta_recur_sm100(recs, gcs, bf, (int64_t)B * H * NC, init2, o, nullptr, T, H, NC, n2, m2, VarLen{}, st);
  }
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
