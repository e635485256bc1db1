// Host side of the TMA path: cuTensorMapEncodeTiled through the runtime's driver entry point.
#include "sm100.cuh"
#include "common.cuh"

#include <algorithm>
#include <mutex>

namespace atma {

PFN_encodeTiled get_encode_tiled() {
  static PFN_encodeTiled fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<PFN_encodeTiled>(p);
  });
  return fn;
}

int make_tmap_16bit_4d(CUtensorMap* out, const void* base, int is_bf16, const uint64_t dims_in[4],
                       const int64_t strides_in[3], const uint32_t box_in[4]) {
  PFN_encodeTiled enc = get_encode_tiled();
  if (enc == nullptr) return fail(ATMA_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
  cuuint64_t dims[4] = {dims_in[0], dims_in[1], dims_in[2], dims_in[3]};
  cuuint64_t strides[3] = {(cuuint64_t)strides_in[0] * 2, (cuuint64_t)strides_in[1] * 2, (cuuint64_t)strides_in[2] * 2};
  cuuint32_t box[4] = {box_in[0], box_in[1], box_in[2], box_in[3]};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = enc(out, is_bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4,
                   const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(ATMA_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
  return ATMA_OK;
}

}  // namespace atma
