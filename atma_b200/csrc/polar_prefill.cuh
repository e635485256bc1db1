// Internal: the two implementations behind atma_polar_prefill.
#pragma once
#include "common.cuh"

namespace atma {

// fp32 CUDA-core kernel: any supported dtype, dk in {32,64,128,256}.
int polar_prefill_simt(const atma_polar_prefill_args& a, cudaStream_t st);

// tcgen05 / TMEM / TMA tile kernel: bf16 or fp16, dk = 128.
bool polar_prefill_sm100_supported(const atma_polar_prefill_args& a);
int polar_prefill_sm100(const atma_polar_prefill_args& a, cudaStream_t st);

}  // namespace atma
