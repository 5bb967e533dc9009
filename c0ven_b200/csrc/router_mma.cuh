// The router's product for steps of many rows, on the tensor cores: approximate logits whose error is bounded, from
// which the top-k kernel picks candidates and recomputes, in the exact order every other path uses, only the logits
// the bound cannot tell apart. It replaces the reference's prompt-path router product (kernels/gemm.cl:51-115, called at
// core/models/qwen4exp/prompt.cpp:608), which is a bf16 product; here the chosen experts must equal an fp32 product's
// bit for bit, so the operands keep 22 bits: each fp32 number is the sum of two f16 numbers, hi + lo, and
//   x . w  ~=  xhi . whi + xhi . wlo + xlo . whi        (the dropped xlo . wlo is 2^-22 of the product)
// as three f16 MMAs into one f32 accumulator. The router's rows are scaled by a power of two per expert so that their
// lo parts are normal f16 numbers; the scale is taken out again, exactly, when the accumulators are read.
//
// A work item is 128 rows of x by 256 experts (128 in steps too short to give every SM an item of 256); persistent CTAs of six warps take items in turn: one thread issues the
// bulk-tensor copies (x hi and lo: 64 values x 128 rows; the router's hi and lo: 64 values x 256 experts, all in the
// 128-byte-swizzled K-major layout), one issues the MMAs (M 128, N 256, K 16; twelve a stage), four warps read the
// accumulators back and store the logits. Tensor memory holds two accumulators of 256 columns, so the MMAs of item
// i + 1 run while item i drains. No copy is multicast; every wait is bounded, as in the experts' tile kernel.
#pragma once

#include "expert_tiles.cuh"

namespace moe {

constexpr uint32_t kRouterTileRows = 128, kRouterTileExperts = 256, kRouterTileK = 64;
constexpr uint32_t kRouterStages = 2;
constexpr uint32_t kRouterThreads = 192;
constexpr uint32_t kRouterABytes = kRouterTileRows * kRouterTileK * 2, kRouterBBytes = kRouterTileExperts * kRouterTileK * 2;
constexpr uint32_t kRouterStageBytes = 2 * kRouterABytes + 2 * kRouterBBytes;      // 96 KB
constexpr uint32_t kRouterSmemBytes = kRouterStages * kRouterStageBytes + 256 + 1024;  // barriers; room to align to 1024

struct RouterMmaArgs {
  uint32_t T, E, NE;
  uint32_t ne_tile;        // experts an item takes: 256, or 128 when items of 256 would leave SMs without one
  const float *w_unscale;  // [NE]: what an accumulator is multiplied by (the inverse of the expert's power-of-two scale)
  float *logits;           // [T][NE]
  uint32_t *error;         // set non-zero when a wait ran out
};

static __global__ void __launch_bounds__(kRouterThreads, 1)
    k_router_mma(const RouterMmaArgs a, const __grid_constant__ CUtensorMap x_hi, const __grid_constant__ CUtensorMap x_lo,
                 const __grid_constant__ CUtensorMap w_hi, const __grid_constant__ CUtensorMap w_lo) {
  using namespace tc;
  constexpr uint32_t S = kRouterStages, kCols = 512;
  extern __shared__ uint8_t smem_raw[];
  uint8_t *smem = (uint8_t *)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const uint32_t tid = threadIdx.x, warp = tid / 32, lane = tid % 32;
  const uint32_t KT = a.E / kRouterTileK, ne_tile = a.ne_tile, col_tiles = (a.NE + ne_tile - 1) / ne_tile;
  const uint32_t nitems = ((a.T + kRouterTileRows - 1) / kRouterTileRows) * col_tiles;
  if (blockIdx.x >= nitems) return;
  uint64_t *bars = (uint64_t *)(smem + S * kRouterStageBytes);
  const uint32_t bar0 = smem_u32(bars);
  auto full_bar = [&](uint32_t s) { return bar0 + 8 * s; };
  auto empty_bar = [&](uint32_t s) { return bar0 + 8 * (S + s); };
  auto acc_full = [&](uint32_t b) { return bar0 + 8 * (2 * S + b); };
  auto acc_empty = [&](uint32_t b) { return bar0 + 8 * (2 * S + 2 + b); };
  uint32_t *tmem_slot = (uint32_t *)(bars + 2 * S + 4);
  volatile uint32_t *abort = tmem_slot + 1;
  if (tid == 0) {
    for (uint32_t s = 0; s < S; s++) mbar_init(full_bar(s), 1), mbar_init(empty_bar(s), 1);
    for (uint32_t b = 0; b < 2; b++) mbar_init(acc_full(b), 1), mbar_init(acc_empty(b), 4);
    *abort = 0;
    fence_barrier_init();
  }
  if (warp == 1) tmem_alloc(smem_u32(tmem_slot), kCols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  bool ok = true;

  if (warp == 0) {
    // The copy thread. Rows past T and experts past NE read as zeros.
    if (lane == 0) {
      uint32_t li = 0;
      for (uint32_t item = blockIdx.x; item < nitems && ok; item += gridDim.x, li++) {
        const uint32_t row0 = (item / col_tiles) * kRouterTileRows, e0 = (item % col_tiles) * ne_tile;
        for (uint32_t it = 0; it < KT && ok; it++) {
          const uint32_t g = li * KT + it, s = g % S, use_s = g / S;
          if (use_s > 0) ok = mbar_wait(empty_bar(s), (use_s - 1) & 1, abort, a.error);
          if (!ok) break;
          const uint32_t st = smem_u32(smem + s * kRouterStageBytes), k0 = it * kRouterTileK;
          // The router's maps copy 128 experts' rows a box: one or two boxes for each half.
          mbar_arrive_expect(full_bar(s), 2 * kRouterABytes + 2 * ne_tile * kRouterTileK * 2);
          tma_load_rows(st, &x_hi, k0, row0, full_bar(s));
          tma_load_rows(st + kRouterABytes, &x_lo, k0, row0, full_bar(s));
          for (uint32_t e = 0; e < ne_tile; e += 128) {
            tma_load_rows(st + 2 * kRouterABytes + e * kRouterTileK * 2, &w_hi, k0, e0 + e, full_bar(s));
            tma_load_rows(st + 2 * kRouterABytes + kRouterBBytes + e * kRouterTileK * 2, &w_lo, k0, e0 + e, full_bar(s));
          }
        }
      }
      if (!ok) {
        // Copies already issued may still be on their way: give them time to land before the CTA leaves.
        const long long t0 = clock64();
        while (clock64() - t0 < 400000) {
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc = (1u << 4) | ((ne_tile >> 3) << 17) | ((kRouterTileRows >> 4) << 24);
      uint32_t li = 0;
      for (uint32_t item = blockIdx.x; item < nitems && ok; item += gridDim.x, li++) {
        const uint32_t b = li & 1, use_b = li / 2;
        if (use_b > 0) ok = mbar_wait(acc_empty(b), (use_b - 1) & 1, abort, a.error);
        for (uint32_t it = 0; it < KT && ok; it++) {
          const uint32_t g = li * KT + it, s = g % S;
          ok = mbar_wait(full_bar(s), (g / S) & 1, abort, a.error);
          if (!ok) break;
          tc_fence_after();
          const uint32_t st = smem_u32(smem + s * kRouterStageBytes);
          const uint32_t xh = st, xl = st + kRouterABytes, wh = st + 2 * kRouterABytes, wl = wh + kRouterBBytes;
          const uint32_t d = tmem_base + b * kRouterTileExperts;
#pragma unroll
          for (uint32_t k = 0; k < kRouterTileK / 16; k++) {
            const uint64_t dxh = smem_desc_sw128(xh + 32 * k), dwh = smem_desc_sw128(wh + 32 * k);
            mma_f16(d, dxh, dwh, idesc, (it | k) != 0);
            mma_f16(d, dxh, smem_desc_sw128(wl + 32 * k), idesc, 1);
            mma_f16(d, smem_desc_sw128(xl + 32 * k), dwh, idesc, 1);
          }
          mma_commit(empty_bar(s));
        }
        if (ok) mma_commit(acc_full(b));
      }
    }
  } else {
    // Epilogue warps: warp w reads TMEM lanes 32 (w % 4) .., a quarter of the item's rows; a lane is a row, and writes
    // 64 bytes of it at a time.
    const uint32_t q = warp % 4;
    uint32_t li = 0;
    for (uint32_t item = blockIdx.x; item < nitems && ok; item += gridDim.x, li++) {
      const uint32_t row0 = (item / col_tiles) * kRouterTileRows, e0 = (item % col_tiles) * ne_tile;
      const uint32_t b = li & 1, use_b = li / 2;
      ok = mbar_wait(acc_full(b), use_b & 1, abort, a.error);
      if (!ok) break;
      tc_fence_after();
      const uint32_t t = row0 + 32 * q + lane;
      float *out = a.logits + (uint64_t)t * a.NE + e0;
      for (uint32_t c = 0; c < ne_tile / 16; c++) {
        if (e0 + 16 * c >= a.NE) break;
        uint32_t v[16];
        tmem_ld16(tmem_base + ((32 * q) << 16) + b * kRouterTileExperts + 16 * c, v);
        tmem_ld_wait();
        if (t < a.T) {
#pragma unroll
          for (int j = 0; j < 16; j += 4) {
            const float4 u = __ldg((const float4 *)(a.w_unscale + e0 + 16 * c + j));
            *(float4 *)(out + 16 * c + j) = make_float4(__uint_as_float(v[j]) * u.x, __uint_as_float(v[j + 1]) * u.y,
                                                       __uint_as_float(v[j + 2]) * u.z, __uint_as_float(v[j + 3]) * u.w);
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(acc_empty(b));
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    tmem_free(tmem_base, kCols);
  }
}

}  // namespace moe
