#include "tensor_map.h"

#include <cudaTypedefs.h>
#include <cuda_runtime_api.h>

#include <string>

#include "cuda_rt.h"

namespace moe {

static PFN_cuTensorMapEncodeTiled_v12000 tensor_map_encoder() {
  // The encoder is a driver call; its address comes through the runtime, so the library does not link the driver.
  static PFN_cuTensorMapEncodeTiled_v12000 encode = [] {
    void *fn = nullptr;
    cudaDriverEntryPointQueryResult q{};
    const cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q);
    if (e != cudaSuccess || q != cudaDriverEntryPointSuccess || !fn) throw CudaFailure(e == cudaSuccess ? cudaErrorNotSupported : e, "cuTensorMapEncodeTiled is not available");
    return (PFN_cuTensorMapEncodeTiled_v12000)fn;
  }();
  return encode;
}

CUtensorMap make_quants_map(const void *base, uint32_t row_bytes, uint32_t rows, uint32_t nslots, uint64_t slice_bytes, uint32_t box_bytes) {
  if (box_bytes != 64 && box_bytes != 128) throw CudaFailure(cudaErrorInvalidValue, "a quant slot's row is 64 or 128 bytes");
  CUtensorMap m{};
  const cuuint64_t dims[3] = {row_bytes, rows, nslots};
  const cuuint64_t strides[2] = {row_bytes, slice_bytes};
  const cuuint32_t box[3] = {box_bytes, 128, 1};
  const cuuint32_t elem[3] = {1, 1, 1};
  const CUresult r = tensor_map_encoder()(&m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void *>(base), dims, strides, box, elem,
                                          CU_TENSOR_MAP_INTERLEAVE_NONE, box_bytes == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_128B,
                                          CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) throw CudaFailure(cudaErrorInvalidValue, "cuTensorMapEncodeTiled failed with driver error " + std::to_string((int)r));
  return m;
}

CUtensorMap make_rows_map(const void *base, uint64_t rows, uint32_t K, uint32_t box_rows) {
  const auto encode = tensor_map_encoder();
  CUtensorMap m{};
  const cuuint64_t dims[2] = {K, rows};
  const cuuint64_t strides[1] = {(cuuint64_t)K * 2};
  const cuuint32_t box[2] = {64, box_rows};
  const cuuint32_t elem[2] = {1, 1};
  const CUresult r = encode(&m, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void *>(base), dims, strides, box, elem,
                            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) throw CudaFailure(cudaErrorInvalidValue, "cuTensorMapEncodeTiled failed with driver error " + std::to_string((int)r));
  return m;
}

}  // namespace moe
