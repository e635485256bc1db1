// atma_polar_prefill: argument validation and the choice between the tensor-core tile kernel
// (16-bit inputs, head_dim 128) and the fp32 CUDA-core kernel (everything else).
#include "polar_prefill.cuh"

using namespace atma;

static int validate(const atma_polar_prefill_args& a) {
  ATMA_REQUIRE(dtype_ok(a.dtype), "polar_prefill: unsupported dtype %d", a.dtype);
  ATMA_REQUIRE(a.B >= 0 && a.H > 0 && a.Hkv > 0 && a.Tq >= 0 && a.Tk >= 0, "polar_prefill: bad shape");
  ATMA_REQUIRE(a.H % a.Hkv == 0, "polar_prefill: H=%d is not a multiple of Hkv=%d", a.H, a.Hkv);
  ATMA_REQUIRE(a.q && a.k && a.v, "polar_prefill: q, k, v are required");
  ATMA_REQUIRE(a.v_null && a.spg && a.null_base && a.sps && a.beta, "polar_prefill: Polar parameters are required");
  ATMA_REQUIRE(a.window >= 0, "polar_prefill: window must be >= 0");
  if (a.finalize) {
    ATMA_REQUIRE(a.c && a.mag, "polar_prefill: c and mag are required when finalize is set");
  } else {
    ATMA_REQUIRE(a.stats_out_m && a.stats_out_l && a.stats_out_q2 && a.stats_out_s,
                 "polar_prefill: stats_out_* are required when finalize is 0");
  }
  const bool any_in = a.stats_in_m || a.stats_in_l || a.stats_in_q2 || a.stats_in_s;
  const bool all_in = a.stats_in_m && a.stats_in_l && a.stats_in_q2 && a.stats_in_s;
  ATMA_REQUIRE(!any_in || all_in, "polar_prefill: stats_in_* must be given together");
  if (a.n_tiles > 0) {
    ATMA_REQUIRE(a.B == 1, "polar_prefill: packed mode takes B == 1");
    ATMA_REQUIRE(a.tile_seq_start && a.tile_q_start && a.tile_seq_len, "polar_prefill: tile map is required");
    ATMA_REQUIRE(a.finalize && !any_in, "polar_prefill: packed mode does not carry statistics");
    ATMA_REQUIRE(a.key_offset == 0, "polar_prefill: packed mode takes key_offset == 0");
  }
  return ATMA_OK;
}

extern "C" int atma_polar_prefill_path(const atma_polar_prefill_args* args) {
  if (args == nullptr) return 0;
  return polar_prefill_sm100_supported(*args) ? 1 : 0;
}

extern "C" int atma_polar_prefill(const atma_polar_prefill_args* args, void* stream) {
  ATMA_REQUIRE(args != nullptr, "polar_prefill: null args");
  const atma_polar_prefill_args& a = *args;
  int rc = validate(a);
  if (rc != ATMA_OK) return rc;
  if (a.B == 0 || a.Tq == 0) return ATMA_OK;
  if (polar_prefill_sm100_supported(a)) return polar_prefill_sm100(a, (cudaStream_t)stream);
  return polar_prefill_simt(a, (cudaStream_t)stream);
}
