// Instantiates and dispatches k_expert_tiles for one weight type; included by the per-type .cu files with
// EXPERT_TILES_QT set.
#pragma once

#include "expert_tiles.cuh"

namespace moe {

template <int QT, int NMAT>
cudaError_t launch_expert_tiles(const ExpertTilesArgs &a, uint32_t max_tiles, const uint32_t *grid_global, cudaStream_t st) {
  if (a.K % kTileK || a.R % kTileM || max_tiles == 0) return cudaErrorInvalidValue;
  auto kernel = k_expert_tiles<QT, NMAT>;
  const size_t smem = TileSmem<NMAT>::kBytes;
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return e;
  kernel<<<dim3(a.R / kTileM, max_tiles), 288, smem, st>>>(a, grid_global);
  return cudaGetLastError();
}

template cudaError_t launch_expert_tiles<EXPERT_TILES_QT, 1>(const ExpertTilesArgs &, uint32_t, const uint32_t *, cudaStream_t);
template cudaError_t launch_expert_tiles<EXPERT_TILES_QT, 2>(const ExpertTilesArgs &, uint32_t, const uint32_t *, cudaStream_t);

}  // namespace moe
