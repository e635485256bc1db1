// Placeholder translation unit, replaced by the tcgen05 tile kernel.
#include "polar_prefill.cuh"
namespace atma {
bool polar_prefill_sm100_supported(const atma_polar_prefill_args&) { return false; }
int polar_prefill_sm100(const atma_polar_prefill_args&, cudaStream_t) {
  return fail(ATMA_ERR_UNSUPPORTED, "polar_prefill: tensor-core path not built");
}
}  // namespace atma
