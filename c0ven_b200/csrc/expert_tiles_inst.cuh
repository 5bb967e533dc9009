// Instantiates and dispatches k_expert_tiles for one weight type; included by the per-type .cu files with
// EXPERT_TILES_QT set.
#pragma once

#include <algorithm>

#include "cuda_rt.h"
#include "expert_tiles.cuh"

namespace moe {

template <int QT, int NMAT>
cudaError_t launch_expert_tiles(const ExpertTilesArgs &a, const CUtensorMap &act_map, uint32_t max_tiles, const uint32_t *grid_global,
                                const LaunchCtx &ctx, cudaStream_t st) {
  if (a.K % kTileK || a.R % kTileM || max_tiles == 0) return cudaErrorInvalidValue;
  auto kernel = k_expert_tiles<QT, NMAT>;
  const size_t smem = TileSmem<QT, NMAT>::kBytes;
  static std::atomic<uint32_t> attr_done{0};
  const cudaError_t e = ensure_dynamic_smem(kernel, smem, attr_done, ctx.device);
  if (e != cudaSuccess) return e;
  const uint64_t items = (uint64_t)max_tiles * (a.R / kTileM);
  kernel<<<(unsigned)std::min<uint64_t>(items, (uint64_t)ctx.sms), kTileThreads, smem, st>>>(a, act_map, grid_global);
  return cudaGetLastError();
}

template cudaError_t launch_expert_tiles<EXPERT_TILES_QT, 1>(const ExpertTilesArgs &, const CUtensorMap &, uint32_t, const uint32_t *, const LaunchCtx &,
                                                             cudaStream_t);
template cudaError_t launch_expert_tiles<EXPERT_TILES_QT, 2>(const ExpertTilesArgs &, const CUtensorMap &, uint32_t, const uint32_t *, const LaunchCtx &,
                                                             cudaStream_t);

}  // namespace moe
