// Instantiates and dispatches k_expert_rows for one weight type; included by the per-type .cu files with
// EXPERT_ROWS_QT set, so that the types compile side by side.
#pragma once

#include "cuda_rt.h"
#include "expert_rows.cuh"

namespace moe {

template <int QT, int NMAT, int M, int G, int UPL>
static cudaError_t launch_one(ExpertRowsArgs a, uint32_t max_groups, const uint32_t *grid_global, const LaunchCtx &ctx, cudaStream_t st) {
  constexpr bool q8k = act_is_q8k(QT);
  // With the row length known at compile time a CTA's eight warps take one batch of passes each; else the caller's count.
  constexpr uint32_t rpp = 32 / G;
  if (UPL > 0)
    a.rows_per_cta = 8 * rpp * rows_batch(NMAT, UPL, M, grid_words(QT) > 0);
  else if (a.rows_per_cta < 8 * rpp)
    a.rows_per_cta = 8 * rpp;
  const size_t smem = (size_t)M * act_row_stride(q8k, a.K) + 4 * grid_words(QT);
  auto kernel = k_expert_rows<QT, NMAT, M, G, UPL>;
  if (smem > 48 * 1024) {
    // The most a group's rows take, whatever this launch's row length: set once per device.
    static std::atomic<uint32_t> attr_done{0};
    const size_t most = (size_t)M * act_row_stride(q8k, kRowsMaxK) + 4 * grid_words(QT);
    if (smem > most) return cudaErrorInvalidValue;
    const cudaError_t e = ensure_dynamic_smem(kernel, most, attr_done, ctx.device);
    if (e != cudaSuccess) return e;
  }
  if (max_groups > 65535) return cudaErrorInvalidValue;  // the grid's second extent; the layer refuses such sizes at create
  // Slabs per CTA: four when that still leaves two CTAs for every CTA slot of the GPU (eight slots an SM), else two,
  // else one. Measured on 32 rows of Q8_0 (247 experts): gate/up 0.142 ms with one slab a CTA, 0.112 with four, 0.119 with eight.
  uint32_t slabs = 1;
  if (UPL > 0) {
    const uint64_t ctas = (uint64_t)((a.R + a.rows_per_cta - 1) / a.rows_per_cta) * max_groups, slots = 8ull * ctx.sms;
    slabs = ctas >= 4 * slots ? 4 : ctas >= 2 * slots ? 2 : 1;
  }
  a.slabs = slabs;
  const dim3 grid((a.R + a.rows_per_cta * slabs - 1) / (a.rows_per_cta * slabs), max_groups);
  return launch_kernel(ctx.pdl, kernel, grid, dim3(256), smem, st, a, grid_global);
}

template <int QT, int NMAT, int M>
static cudaError_t launch_shape(const ExpertRowsArgs &a, uint32_t max_groups, const uint32_t *grid_global, const LaunchCtx &ctx, cudaStream_t st) {
  const uint32_t upr = a.K / Unit<QT>::kValues;
  // The three row lengths the kernels are specialised for are 2048, 512 and 256 values; any other takes the general
  // instantiation, which finds a row's units at run time.
  constexpr uint32_t U2048 = 2048 / Unit<QT>::kValues, U512 = 512 / Unit<QT>::kValues, U256 = 256 / Unit<QT>::kValues;
  if (upr == U2048) return launch_one<QT, NMAT, M, 32, U2048 / 32>(a, max_groups, grid_global, ctx, st);
  // A row of 32 units (Q8_0's 512 values): 16 lanes with two units each, two rows a warp pass, so that a reduction and a
  // store serve twice the bytes.
  if (upr == U512) return launch_one<QT, NMAT, M, (U512 < 32 ? U512 : 16), (U512 < 32 ? 1 : U512 / 16)>(a, max_groups, grid_global, ctx, st);
  if (upr == U256) return launch_one<QT, NMAT, M, (U256 < 32 ? U256 : 32), 1>(a, max_groups, grid_global, ctx, st);
  return launch_one<QT, NMAT, M, 32, 0>(a, max_groups, grid_global, ctx, st);
}

template <int QT, int NMAT>
cudaError_t launch_expert_rows(const ExpertRowsArgs &a, int M, uint32_t max_groups, const uint32_t *grid_global, const LaunchCtx &ctx, cudaStream_t st) {
  switch (M) {
    case 1: return launch_shape<QT, NMAT, 1>(a, max_groups, grid_global, ctx, st);
    case 2: return launch_shape<QT, NMAT, 2>(a, max_groups, grid_global, ctx, st);
    case 4: return launch_shape<QT, NMAT, 4>(a, max_groups, grid_global, ctx, st);
    case 8: return launch_shape<QT, NMAT, 8>(a, max_groups, grid_global, ctx, st);
    default: return cudaErrorInvalidValue;
  }
}

template cudaError_t launch_expert_rows<EXPERT_ROWS_QT, 1>(const ExpertRowsArgs &, int, uint32_t, const uint32_t *, const LaunchCtx &, cudaStream_t);
template cudaError_t launch_expert_rows<EXPERT_ROWS_QT, 2>(const ExpertRowsArgs &, int, uint32_t, const uint32_t *, const LaunchCtx &, cudaStream_t);

}  // namespace moe
