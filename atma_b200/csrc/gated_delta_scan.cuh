// Shared between the gated-delta scan kernels (16-bit inputs, d_k = d_v = 128, chunk = 64): the
// per-chunk factor record that the chunk-local kernel writes and the recurrence kernels read, and
// the descriptors of packed ("varlen") batches and of recurrence-to-factor maps.
#pragma once

#include <cstdint>

namespace atma {
namespace scan {

constexpr int kC = 64, kD = 128;
// One record per (sequence, head, chunk), 16-bit row-major tiles: three [64 rows][128 k], then U0
// transposed [128 v][64 rows], then [64][64]:
//   -W = -T diag(beta g) K | Qg = diag(g) Q | Kt = diag(g_C / g) K | U0^T = (T diag(beta) V)^T | Rq = tril((g_p/g_s) q_p.k_s)
constexpr int kRecW = 0, kRecQg = kC * kD * 2, kRecKt = 2 * kC * kD * 2, kRecU0 = 3 * kC * kD * 2,
              kRecRq = 4 * kC * kD * 2, kRecBytes = 4 * kC * kD * 2 + kC * kC * 2;    // 73,728 B per chunk

// Packed batches: sequences of different lengths back to back in one token axis.  Chunks never
// straddle sequences: sequence i owns chunk records cu_chunks[i] .. cu_chunks[i+1]-1.
struct VarLen {
  const int32_t* cu_seqlens;   // device [n_seqs + 1] token offsets; nullptr = dense (B, T) batch
  const int32_t* cu_chunks;    // device [n_seqs + 1] chunk offsets (built by varlen_chunk_offsets_kernel)
  int n_seqs;
  const int64_t* slots;        // device [n_seqs] rows of state_table, or nullptr (dense state arrays)
  const int32_t* has_initial;  // device [n_seqs] or nullptr (= every sequence starts from its table row)
  float* state_table;          // [rows][H][dk][dv] fp32, or nullptr
  int64_t slot_stride;         // elements between table rows
  // state snapshots for prefix reuse: after every snap_chunks chunks that lie wholly inside the
  // sequence, the fp32 state goes to snapshots[snap_offsets[seq] + j] ([...][H][dk][dv]); nullptr = none
  float* snapshots;
  const int32_t* snap_offsets; // device [n_seqs]
  int snap_chunks;
};

constexpr int kMaxRec = 64;   // recurrences per launch
struct RecMap {                 // recurrence i walks the chunk records of batch entry rec[i];
  int rec[kMaxRec];             // zero_u0[i] != 0 replaces U0 by zero (the "v = 0" recurrence that
  int zero_u0[kMaxRec];         // yields a segment's state-transfer matrix)
  int c_begin[kMaxRec];         // chunk range [c_begin, c_end) of the records that recurrence i walks
  int c_end[kMaxRec];           // (c_end = 0 means "all NC chunks")
  int o_row[kMaxRec];           // batch row of the output tensor that recurrence i writes (negative: no output)
  int state_row[kMaxRec];       // plane of initial_state / final_state that recurrence i reads / writes
};

}  // namespace scan

// Recurrence over the chunk records on the 5th-generation tensor cores (gated_delta_scan_sm100.cu).
// Dense form: n_rec recurrences over the records of a scratch built for B sequences of T tokens;
// packed form (var.cu_seqlens != nullptr): one recurrence per sequence.  o may be null (state only).
int gated_delta_recur_sm100(const uint8_t* recs, const float* gcs, int is_bf16, int64_t n_records, const float* initial_state,
                            void* o, float* final_state, int Tlen, int H, int NC, int n_rec, const scan::RecMap& map,
                            const scan::VarLen& var, cudaStream_t st);
int scan_sm100_status_fetch_and_clear(int* out);

// Chunk-local factors on the 5th-generation tensor cores (gated_delta_local_sm100.cu): q (tokens, H, 128),
// k, v (tokens, Hkv, 128) contiguous 16-bit; g, beta (tokens, H) fp32; records and g_C as laid out above.
// Dense form: B sequences of Tlen tokens (NC chunks each); packed form: var.cu_seqlens / cu_chunks.
int gated_delta_local_sm100(const void* q, const void* k, const void* v, int is_bf16, const float* g, const float* beta,
                            uint8_t* recs, float* gcs, int B, int Tlen, int H, int Hkv, int NC, int normalize_qk, float scale,
                            const scan::VarLen& var, int64_t total_tokens, cudaStream_t st);
int scan_local_status_fetch_and_clear(int* out);

}  // namespace atma
