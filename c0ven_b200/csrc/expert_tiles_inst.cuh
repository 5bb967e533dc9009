// Instantiates and dispatches k_expert_tiles for one weight type; included by the per-type .cu files with
// EXPERT_TILES_QT set.
#pragma once

#include <algorithm>

#include "cuda_rt.h"
#include "expert_tiles.cuh"

namespace moe {

// Pairs of CTAs the GPU runs at once for kernel (one CTA an SM, so at most one pair a TPC), asked once per device.
template <class Kernel>
static cudaError_t max_pairs(Kernel kernel, size_t smem, int device, uint32_t &pairs) {
  static std::atomic<uint32_t> known[64];
  if (device < 0 || device >= 64) return cudaErrorInvalidValue;
  pairs = known[device].load(std::memory_order_acquire);
  if (pairs) return cudaSuccess;
  cudaLaunchConfig_t cfg{};
  cudaLaunchAttribute at{};
  at.id = cudaLaunchAttributeClusterDimension;
  at.val.clusterDim.x = 2, at.val.clusterDim.y = 1, at.val.clusterDim.z = 1;
  cfg.gridDim = dim3(2), cfg.blockDim = dim3(kTileThreads), cfg.dynamicSmemBytes = smem, cfg.attrs = &at, cfg.numAttrs = 1;
  int n = 0;
  const cudaError_t e = cudaOccupancyMaxActiveClusters(&n, kernel, &cfg);
  if (e != cudaSuccess) return e;
  if (n <= 0) return cudaErrorInvalidConfiguration;
  pairs = (uint32_t)n;
  known[device].store(pairs, std::memory_order_release);
  return cudaSuccess;
}

template <int QT, int NMAT>
cudaError_t launch_expert_tiles(const ExpertTilesArgs &a, const CUtensorMap &act_map, uint32_t max_tiles, const uint32_t *grid_global,
                                const LaunchCtx &ctx, cudaStream_t st) {
  if (a.K % kTileK || a.R % kTileM || max_tiles == 0) return cudaErrorInvalidValue;
  const uint32_t RT = a.R / kTileM;
  if (RT % 2 == 0) {
    // Pairs of CTAs on 256 weight rows an item: half the rows' bytes through each CTA's shared memory.
    auto kernel = k_expert_tiles<QT, NMAT, true>;
    const size_t smem = TileSmem<QT, NMAT, true>::kBytes;
    static std::atomic<uint32_t> attr_done{0};
    cudaError_t e = ensure_dynamic_smem(kernel, smem, attr_done, ctx.device);
    if (e != cudaSuccess) return e;
    uint32_t pairs = 0;
    e = max_pairs(kernel, smem, ctx.device, pairs);
    if (e != cudaSuccess) return e;
    const uint64_t items = (uint64_t)max_tiles * (RT / 2);
    cudaLaunchConfig_t cfg{};
    cudaLaunchAttribute at{};
    at.id = cudaLaunchAttributeClusterDimension;
    at.val.clusterDim.x = 2, at.val.clusterDim.y = 1, at.val.clusterDim.z = 1;
    cfg.gridDim = dim3(2 * (unsigned)std::min<uint64_t>(items, pairs)), cfg.blockDim = dim3(kTileThreads);
    cfg.dynamicSmemBytes = smem, cfg.stream = st, cfg.attrs = &at, cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, a, act_map, grid_global);
  }
  auto kernel = k_expert_tiles<QT, NMAT, false>;
  const size_t smem = TileSmem<QT, NMAT, false>::kBytes;
  static std::atomic<uint32_t> attr_done{0};
  const cudaError_t e = ensure_dynamic_smem(kernel, smem, attr_done, ctx.device);
  if (e != cudaSuccess) return e;
  const uint64_t items = (uint64_t)max_tiles * RT;
  kernel<<<(unsigned)std::min<uint64_t>(items, (uint64_t)ctx.sms), kTileThreads, smem, st>>>(a, act_map, grid_global);
  return cudaGetLastError();
}

template cudaError_t launch_expert_tiles<EXPERT_TILES_QT, 1>(const ExpertTilesArgs &, const CUtensorMap &, uint32_t, const uint32_t *, const LaunchCtx &,
                                                             cudaStream_t);
template cudaError_t launch_expert_tiles<EXPERT_TILES_QT, 2>(const ExpertTilesArgs &, const CUtensorMap &, uint32_t, const uint32_t *, const LaunchCtx &,
                                                             cudaStream_t);

}  // namespace moe
