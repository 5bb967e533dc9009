// The block's routing and elementwise stages: activation quantisers, router logits, top-k with renormalised weights,
// the stable pack into expert order with its tiles and groups, and the weighted combine. They replace the reference's
// quantize_a8 (kernels/include/a8.h:9-16), the router product (kernels/common.cl:114-158, kernels/gemm.cl:51-115),
// router / p_router (kernels/models/qwen4exp/layer.cl:765-847, prompt.cl:652-678, route.h:39-98), p_moe_count / scan /
// fill (prompt.cl:682-738), moe_group (layer.cl:894-978) and moe_combine / p_moe_combine (layer.cl:869-883,
// prompt.cl:769-786).
#pragma once

#include <cuda_runtime.h>

#include <cstdint>

#include "expert_rows.cuh"
#include "expert_tiles.cuh"

namespace moe {

struct MoeTile {
  uint32_t expert, slot, start, count;
};
constexpr uint32_t kTileRows = 64;      // MOE_TILE (shared/moe_tile.h:9)
constexpr uint32_t kChunkTokens = 32;   // rows one CTA of the top-k kernel routes: a chunk of the pack
constexpr uint32_t kRouterPieces = 8;   // pieces a router product is summed in

// ---------------------------------------------------------------------------------------------------------------
// Activation quantisers. One warp per 256 values.

// q8_0: per 32 values d = max|x| / 127, q = round(x * (1 / d)), 0 when d is 0; d kept as the f16 the CPU stores
// (docs/spec/QUANT_FORMATS.md:463-465, :525-526).
// With gate set (a vector of `per_row` * 256 floats), a block of 256 values also leaves its part of the row's product
// with the vector in gate_parts[block]: the shared expert's gate logit, summed by the top-k kernel.
__device__ __forceinline__ void gate_part(const float4 &a, const float4 &b, const float *gate, uint32_t per_row, uint64_t blk,
                                          uint32_t lane, float *gate_parts) {
  const float4 *g = (const float4 *)(gate + (blk % per_row) * 256);
  const float4 ga = g[2 * lane], gb = g[2 * lane + 1];
  float s = a.x * ga.x + a.y * ga.y + a.z * ga.z + a.w * ga.w + b.x * gb.x + b.y * gb.y + b.z * gb.z + b.w * gb.w;
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
  if (lane == 0) gate_parts[blk] = s;
}

static __global__ void __launch_bounds__(256) k_quant_q8_0(const float *__restrict__ x, uint64_t nblk256, int8_t *__restrict__ q,
                                                   float *__restrict__ d, __half *__restrict__ deq, const float *__restrict__ gate,
                                                   uint32_t per_row, float *__restrict__ gate_parts) {
  const uint64_t blk = (uint64_t)blockIdx.x * 8 + threadIdx.x / 32;
  if (blk >= nblk256) return;
  const uint32_t lane = threadIdx.x % 32;
  const float4 a = ((const float4 *)(x + blk * 256))[2 * lane], b = ((const float4 *)(x + blk * 256))[2 * lane + 1];
  if (gate) gate_part(a, b, gate, per_row, blk, lane, gate_parts);
  float amax = fmaxf(fmaxf(fmaxf(fabsf(a.x), fabsf(a.y)), fmaxf(fabsf(a.z), fabsf(a.w))),
                     fmaxf(fmaxf(fabsf(b.x), fabsf(b.y)), fmaxf(fabsf(b.z), fabsf(b.w))));
  amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
  amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));  // 4 lanes hold a block of 32
  const float dd = amax / 127.0f, id = dd != 0.0f ? 1.0f / dd : 0.0f;
  char4 lo, hi;
  lo.x = (signed char)roundf(a.x * id), lo.y = (signed char)roundf(a.y * id);
  lo.z = (signed char)roundf(a.z * id), lo.w = (signed char)roundf(a.w * id);
  hi.x = (signed char)roundf(b.x * id), hi.y = (signed char)roundf(b.y * id);
  hi.z = (signed char)roundf(b.z * id), hi.w = (signed char)roundf(b.w * id);
  ((char4 *)(q + blk * 256))[2 * lane] = lo;
  ((char4 *)(q + blk * 256))[2 * lane + 1] = hi;
  const float dh = __half2float(__float2half_rn(dd));
  if (lane % 4 == 0) d[blk * 8 + lane / 4] = dh;
  if (deq) {  // the codes dequantised, as f16: what the tensor-core kernels take for this row
    const __half2 h0 = __floats2half2_rn(dh * (float)lo.x, dh * (float)lo.y), h1 = __floats2half2_rn(dh * (float)lo.z, dh * (float)lo.w);
    const __half2 h2 = __floats2half2_rn(dh * (float)hi.x, dh * (float)hi.y), h3 = __floats2half2_rn(dh * (float)hi.z, dh * (float)hi.w);
    uint4 o;
    o.x = *(const uint32_t *)&h0, o.y = *(const uint32_t *)&h1, o.z = *(const uint32_t *)&h2, o.w = *(const uint32_t *)&h3;
    ((uint4 *)(deq + blk * 256))[lane] = o;
  }
}

// q8_K: per 256 values iscale = -127 / max with max the value of largest magnitude (the first of equals),
// q = min(127, nearest-even(iscale * x)), d = 1 / iscale, and the sums of each 16 codes (QUANT_FORMATS.md:528-535).
static __global__ void __launch_bounds__(256) k_quant_q8_K(const float *__restrict__ x, uint64_t nblk256, int8_t *__restrict__ q,
                                                   float *__restrict__ d, int16_t *__restrict__ bs, __half *__restrict__ deq,
                                                   const float *__restrict__ gate, uint32_t per_row, float *__restrict__ gate_parts) {
  const uint64_t blk = (uint64_t)blockIdx.x * 8 + threadIdx.x / 32;
  if (blk >= nblk256) return;
  const uint32_t lane = threadIdx.x % 32;
  const float4 a = ((const float4 *)(x + blk * 256))[2 * lane], b = ((const float4 *)(x + blk * 256))[2 * lane + 1];
  if (gate) gate_part(a, b, gate, per_row, blk, lane, gate_parts);
  const float v[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
  float amax = 0.0f, mx = 0.0f;
  uint32_t at = 8 * lane;
#pragma unroll
  for (int i = 0; i < 8; i++)
    if (fabsf(v[i]) > amax) amax = fabsf(v[i]), mx = v[i], at = 8 * lane + i;
#pragma unroll
  for (int off = 1; off < 32; off <<= 1) {
    const float oa = __shfl_xor_sync(0xffffffffu, amax, off), om = __shfl_xor_sync(0xffffffffu, mx, off);
    const uint32_t oat = __shfl_xor_sync(0xffffffffu, at, off);
    if (oa > amax || (oa == amax && oat < at)) amax = oa, mx = om, at = oat;
  }
  if (amax == 0.0f) {
    ((char4 *)(q + blk * 256))[2 * lane] = make_char4(0, 0, 0, 0);
    ((char4 *)(q + blk * 256))[2 * lane + 1] = make_char4(0, 0, 0, 0);
    if (lane == 0) d[blk] = 0.0f;
    if (lane % 2 == 0) bs[blk * 16 + lane / 2] = 0;
    if (deq) ((uint4 *)(deq + blk * 256))[lane] = make_uint4(0, 0, 0, 0);
    return;
  }
  const float iscale = -127.0f / mx;
  int c[8], sum = 0;
#pragma unroll
  for (int i = 0; i < 8; i++) c[i] = min(127, __float2int_rn(__fmul_rn(iscale, v[i]))), sum += c[i];
  ((char4 *)(q + blk * 256))[2 * lane] = make_char4((signed char)c[0], (signed char)c[1], (signed char)c[2], (signed char)c[3]);
  ((char4 *)(q + blk * 256))[2 * lane + 1] = make_char4((signed char)c[4], (signed char)c[5], (signed char)c[6], (signed char)c[7]);
  sum += __shfl_xor_sync(0xffffffffu, sum, 1);
  if (lane % 2 == 0) bs[blk * 16 + lane / 2] = (int16_t)sum;
  const float dd = 1.0f / iscale;
  if (lane == 0) d[blk] = dd;
  if (deq) {
    const __half2 h0 = __floats2half2_rn(dd * (float)c[0], dd * (float)c[1]), h1 = __floats2half2_rn(dd * (float)c[2], dd * (float)c[3]);
    const __half2 h2 = __floats2half2_rn(dd * (float)c[4], dd * (float)c[5]), h3 = __floats2half2_rn(dd * (float)c[6], dd * (float)c[7]);
    uint4 o;
    o.x = *(const uint32_t *)&h0, o.y = *(const uint32_t *)&h1, o.z = *(const uint32_t *)&h2, o.w = *(const uint32_t *)&h3;
    ((uint4 *)(deq + blk * 256))[lane] = o;
  }
}

// ---------------------------------------------------------------------------------------------------------------
// Router logits: rl[t][e] = W[e] . x[t] for the NE experts and, as row NE, the shared expert's gate vector. Every
// product is summed in kRouterPieces equal pieces of the row, each a chain of fused multiply-adds from 0 in index
// order, the pieces then added in order, and an expert's bias last. Both kernels and the CPU oracle keep this one
// order, so that the logits, and with them the chosen experts, agree bit for bit whatever the row count.

// Few rows (up to TM per CTA pass): a warp takes 4 weight rows, 8 lanes a row, lane s taking piece s; D loads of 16 bytes
// in flight per lane (a piece is a multiple of 4 D values: 8 always, 16 when the piece is a multiple of 64 values). A CTA is one warp when the step has one or two rows, so that
// the router's 4 MB spread over 129 CTAs, and eight warps otherwise, so that the staged rows serve 32 weight rows.
template <int TM, int D = 8>
static __global__ void __launch_bounds__(256) k_router_logits_rows(const float *__restrict__ x, uint32_t T, uint32_t E,
                                                          const float *__restrict__ W, uint32_t N,
                                                          const float *__restrict__ bias, uint32_t NE,
                                                          float *__restrict__ rl) {
  extern __shared__ __align__(16) float xs[];  // TM rows, each piece padded by 4 floats to spread the banks
  const uint32_t piece = E / kRouterPieces, pstride = piece + 4, rstride = kRouterPieces * pstride;
  const uint32_t t0 = blockIdx.y * TM, tn = min((uint32_t)TM, T - t0);
  const uint32_t lane = threadIdx.x % 32, s = lane % 8, row = (blockIdx.x * (blockDim.x / 32) + threadIdx.x / 32) * 4 + lane / 8;
  // The first weights are on their way while the rows are staged.
  const float4 *w = (const float4 *)(W + (uint64_t)min(row, N - 1) * E + s * piece);
  float4 wq[D];
#pragma unroll
  for (int i = 0; i < D; i++) wq[i] = __ldg(w + i);
  for (uint32_t i = threadIdx.x; i < TM * (E / 4); i += blockDim.x) {
    const uint32_t t = i / (E / 4), k4 = i % (E / 4), k = 4 * k4;
    const float4 v = t < tn ? ((const float4 *)(x + (uint64_t)(t0 + t) * E))[k4] : make_float4(0, 0, 0, 0);
    *(float4 *)(xs + t * rstride + (k / piece) * pstride + k % piece) = v;
  }
  __syncthreads();
  float p[TM];
#pragma unroll
  for (int t = 0; t < TM; t++) p[t] = 0.0f;
  const float *xp = xs + s * pstride;
  for (uint32_t i0 = 0; i0 < piece / 4; i0 += D) {
    float4 cur[D];
#pragma unroll
    for (int i = 0; i < D; i++) cur[i] = wq[i];
    if (i0 + D < piece / 4) {
#pragma unroll
      for (int i = 0; i < D; i++) wq[i] = __ldg(w + i0 + D + i);
    }
#pragma unroll
    for (int i = 0; i < D; i++) {
#pragma unroll
      for (int t = 0; t < TM; t++) {
        const float4 xv = *(const float4 *)(xp + t * rstride + 4 * (i0 + i));
        p[t] = fmaf(xv.x, cur[i].x, p[t]);
        p[t] = fmaf(xv.y, cur[i].y, p[t]);
        p[t] = fmaf(xv.z, cur[i].z, p[t]);
        p[t] = fmaf(xv.w, cur[i].w, p[t]);
      }
    }
  }
#pragma unroll
  for (int t = 0; t < TM; t++) {
    float tot = __shfl_sync(0xffffffffu, p[t], lane & ~7u);
#pragma unroll
    for (int j = 1; j < (int)kRouterPieces; j++) tot = __fadd_rn(tot, __shfl_sync(0xffffffffu, p[t], (lane & ~7u) + j));
    if (s == 0 && row < N && (uint32_t)t < tn) {
      if (bias && row < NE) tot = __fadd_rn(tot, bias[row]);
      rl[(uint64_t)(t0 + t) * N + row] = tot;
    }
  }
}

// Many rows: the product piece by piece. A CTA takes a 128 x 128 (or 96 x 128) tile of (rows, experts) and one of the kRouterPieces
// pieces of the hidden size, 8 x 8 outputs a thread, 16 values of the piece a step, each output one chain of fused
// multiply-adds in index order; it leaves the piece's partial sums in P[piece][row][expert]. The top-k kernel adds a
// row's pieces in order. Splitting by piece gives eight times the CTAs, which keeps every SM busy at a few thousand
// rows, and frees the registers the running totals would take. The shared expert's gate logit does not come from
// here: the activation quantiser sums it (k_quant_*'s gate argument).
template <int RM>
static __global__ void __launch_bounds__(256, 2) k_router_pieces(const float *__restrict__ x, uint32_t T, uint32_t E,
                                                                const float *__restrict__ W, uint32_t NE, float *__restrict__ P) {
  constexpr int BM = RM == 8 ? 128 : 96, BN = 128, BK = 16, LD = 128 + 4;
  static_assert(RM == 8 || RM == 6, "tiles of 128 or 96 rows");
  __shared__ __align__(16) float As[2][BK][LD], Bs[2][BK][LD];
  const uint32_t tid = threadIdx.x, ty = tid / 16, tx = tid % 16;
  const uint32_t m0 = blockIdx.y * BM, n0 = blockIdx.x * BN, piece = E / kRouterPieces, kbeg = blockIdx.z * piece;
  float acc[RM][8];
#pragma unroll
  for (int i = 0; i < RM; i++)
#pragma unroll
    for (int j = 0; j < 8; j++) acc[i][j] = 0.0f;
  // A thread's loads per step: two float4 of x and two of W, rows lr and the quarter lq of the step's 16 values and the
  // one two on. A warp's lanes hold consecutive rows, so the transposed stores fill consecutive banks.
  const uint32_t lr = tid % 128, lq = tid / 128;
  float4 ra[2], rb[2];
  auto fetch = [&](uint32_t k0) {
    const uint32_t r = m0 + lr, e = n0 + lr;
#pragma unroll
    for (int i = 0; i < 2; i++) {
      ra[i] = (lr < BM && r < T) ? __ldg((const float4 *)(x + (uint64_t)r * E + k0 + 4 * (lq + 2 * i))) : make_float4(0, 0, 0, 0);
      rb[i] = e < NE ? __ldg((const float4 *)(W + (uint64_t)e * E + k0 + 4 * (lq + 2 * i))) : make_float4(0, 0, 0, 0);
    }
  };
  auto stash = [&](int buf) {
#pragma unroll
    for (int i = 0; i < 2; i++) {
      const uint32_t k = 4 * (lq + 2 * i);
      As[buf][k + 0][lr] = ra[i].x, As[buf][k + 1][lr] = ra[i].y, As[buf][k + 2][lr] = ra[i].z, As[buf][k + 3][lr] = ra[i].w;
      Bs[buf][k + 0][lr] = rb[i].x, Bs[buf][k + 1][lr] = rb[i].y, Bs[buf][k + 2][lr] = rb[i].z, Bs[buf][k + 3][lr] = rb[i].w;
    }
  };
  fetch(kbeg);
  stash(0);
  __syncthreads();
  const uint32_t steps = piece / BK;
  for (uint32_t s = 0; s < steps; s++) {
    const int buf = s & 1;
    if (s + 1 < steps) fetch(kbeg + (s + 1) * BK);
#pragma unroll
    for (int k = 0; k < BK; k++) {
      // A thread's rows: ty * 4 .. + 3 and, past row 64, ty * 4 .. + 3 again (128-row tiles) or ty * 2, ty * 2 + 1 (96).
      const float4 a0 = *(const float4 *)&As[buf][k][ty * 4];
      float av[RM] = {a0.x, a0.y, a0.z, a0.w};
      if constexpr (RM == 8) {
        const float4 a1 = *(const float4 *)&As[buf][k][64 + ty * 4];
        av[4] = a1.x, av[5] = a1.y, av[6] = a1.z, av[7] = a1.w;
      } else {
        const float2 a1 = *(const float2 *)&As[buf][k][64 + ty * 2];
        av[4] = a1.x, av[5] = a1.y;
      }
      const float4 b0 = *(const float4 *)&Bs[buf][k][tx * 4], b1 = *(const float4 *)&Bs[buf][k][64 + tx * 4];
      const float bv[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
      for (int i = 0; i < RM; i++)
#pragma unroll
        for (int j = 0; j < 8; j++) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
    }
    if (s + 1 < steps) stash(buf ^ 1);
    __syncthreads();
  }
  float *out = P + (uint64_t)blockIdx.z * T * NE;
#pragma unroll
  for (int i = 0; i < RM; i++) {
    const uint32_t t = m0 + (i < 4 ? ty * 4 + i : 64 + ty * (RM - 4) + i - 4);
    if (t >= T) continue;
#pragma unroll
    for (int h = 0; h < 2; h++) {
      const uint32_t e = n0 + 64 * h + tx * 4;
      if (e + 3 < NE)
        *(float4 *)(out + (uint64_t)t * NE + e) = make_float4(acc[i][4 * h], acc[i][4 * h + 1], acc[i][4 * h + 2], acc[i][4 * h + 3]);
      else
        for (int j = 0; j < 4; j++)
          if (e + j < NE) out[(uint64_t)t * NE + e + j] = acc[i][4 * h + j];
    }
  }
}

// Rows a thread of k_router_pieces takes (8: tiles of 128 rows, 6: of 96) for T rows on a GPU that holds `slots` of its
// CTAs at once: the height whose whole waves cost less. 3,521 rows in tiles of 128 are 896 CTAs, three waves of 296 and
// eight CTAs of a fourth; in tiles of 96, 1,184 CTAs, four waves three quarters as long.
inline int router_rows_per_thread(uint32_t T, uint32_t NE, uint32_t slots) {
  auto cost = [&](int rm) {
    const uint64_t ctas = (uint64_t)((T + 16 * rm - 1) / (16 * rm)) * ((NE + 127) / 128) * kRouterPieces;
    return ((ctas + slots - 1) / slots) * rm;
  };
  // A 96-row tile does 48 multiply-adds for the shared-memory loads that feed 64 in a 128-row tile: measured, a row
  // costs it about a fifth more (3,521 rows: 0.257 -> 0.236 ms; 32,768 rows: 1.90 -> 2.03 ms when it was chosen there).
  return cost(6) * 6 < cost(8) * 5 ? 6 : 8;
}

// ---------------------------------------------------------------------------------------------------------------
// Top-k. One warp per row, lane holding experts lane + 32 j. Keys order the logits as floats do (the reference's
// topk_key, kernels/include/topk.h:12-15), -0 taken as +0; winners come out largest first, ties to the lower expert
// (route.h:33-38). Weights: p_k = exp(v_k - max) / sum, w_k = p_k / max(sum of the K p's, 6.1035e-5)
// (layer.cl:784-787). The CTA's rows are one chunk of the pack: it leaves the chunk's count of every expert.
__device__ __forceinline__ uint32_t order_key(float v) {
  const uint32_t u = __float_as_uint(v + 0.0f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ float key_value(uint32_t key) {
  return __uint_as_float((key & 0x80000000u) ? (key & 0x7fffffffu) : ~key);
}

constexpr int kMaxPerLane = 16;  // experts a lane holds at most: 512 / 32

// The logits come as rows rl[t][NE + 1] (the gate's logit last), or, with pieces set, as the partial sums
// pieces[p][t][e] of k_router_pieces, added here in order with the bias, and the gate's logit as gate_parts[t][nparts].
// The block's part: its rows' ids, weights and gates written, the chunk's count of every expert left in hist (shared,
// 512 words) and, when s_ids is not null, the chunk's ids there too (shared, kChunkTokens * K words).
__device__ __forceinline__ void router_topk_block(const float *__restrict__ rl, const float *__restrict__ pieces,
                                                  const float *__restrict__ bias, const float *__restrict__ gate_parts, uint32_t nparts,
                                                  uint32_t T, uint32_t NE, uint32_t K, int32_t *__restrict__ ids, float *__restrict__ w,
                                                  float *__restrict__ gs, uint32_t *hist, int32_t *s_ids) {
  for (uint32_t i = threadIdx.x; i < NE; i += blockDim.x) hist[i] = 0;
  __syncthreads();
  const uint32_t lane = threadIdx.x % 32, t = blockIdx.x * kChunkTokens + threadIdx.x / 32, per = NE / 32;
  if (t < T) {
    uint32_t key[kMaxPerLane];
    float mx = -INFINITY;
#pragma unroll
    for (int j = 0; j < kMaxPerLane; j++) {
      key[j] = 0;
      if ((uint32_t)j < per) {
        const uint32_t e = lane + 32 * j;
        float f;
        if (pieces) {
          f = pieces[(uint64_t)t * NE + e];
#pragma unroll
          for (uint32_t p = 1; p < kRouterPieces; p++) f = __fadd_rn(f, pieces[((uint64_t)p * T + t) * NE + e]);
          if (bias) f = __fadd_rn(f, bias[e]);
        } else {
          f = rl[(uint64_t)t * (NE + 1) + e];
        }
        key[j] = order_key(f);
        mx = fmaxf(mx, f);
      }
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
    float sum = 0.0f;
#pragma unroll
    for (int j = 0; j < kMaxPerLane; j++)
      if ((uint32_t)j < per) sum += expf(key_value(key[j]) - mx);
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
    // K rounds of arg-max over (key, lower expert first).
    float pk = 0.0f;
    uint32_t my_id = 0;
    for (uint32_t k = 0; k < K; k++) {
      unsigned long long best = 0;
#pragma unroll
      for (int j = 0; j < kMaxPerLane; j++) {
        const unsigned long long c = ((unsigned long long)key[j] << 32) | (uint32_t)~(lane + 32 * j);
        if ((uint32_t)j < per && c > best) best = c;
      }
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) {
        const unsigned long long o = __shfl_xor_sync(0xffffffffu, best, off);
        if (o > best) best = o;
      }
      const uint32_t e = ~(uint32_t)best, bkey = (uint32_t)(best >> 32);
      if (e % 32 == lane) {
#pragma unroll
        for (int j = 0; j < kMaxPerLane; j++)
          if ((uint32_t)j == e / 32) key[j] = 0;
      }
      if (lane == k) {
        my_id = e;
        pk = expf(key_value(bkey) - mx) / sum;
      }
    }
    float tot = 0.0f;
    for (uint32_t k = 0; k < K; k++) tot += __shfl_sync(0xffffffffu, pk, k);
    if (lane < K) {
      ids[(uint64_t)t * K + lane] = (int32_t)my_id;
      w[(uint64_t)t * K + lane] = pk / fmaxf(tot, 6.1035e-5f);
      atomicAdd(&hist[my_id], 1u);
      if (s_ids) s_ids[(threadIdx.x / 32) * K + lane] = (int32_t)my_id;
    }
    if (lane == 0) {
      float g;
      if (pieces) {
        g = 0.0f;
        for (uint32_t p = 0; p < nparts; p++) g += gate_parts[(uint64_t)t * nparts + p];
      } else {
        g = rl[(uint64_t)t * (NE + 1) + NE];
      }
      gs[t] = 1.0f / (1.0f + expf(-g));
    }
  }
  __syncthreads();
}

static __global__ void __launch_bounds__(32 * kChunkTokens) k_router_topk(const float *__restrict__ rl, const float *__restrict__ pieces,
                                                                  const float *__restrict__ bias, const float *__restrict__ gate_parts,
                                                                  uint32_t nparts, uint32_t T, uint32_t NE,
                                                                  uint32_t K, int32_t *__restrict__ ids,
                                                                  float *__restrict__ w, float *__restrict__ gs,
                                                                  uint32_t *__restrict__ chunk_hist) {
  __shared__ uint32_t hist[512];
  router_topk_block(rl, pieces, bias, gate_parts, nparts, T, NE, K, ids, w, gs, hist, nullptr);
  for (uint32_t i = threadIdx.x; i < NE; i += blockDim.x) chunk_hist[(uint64_t)blockIdx.x * NE + i] = hist[i];
}

// The same counts for expert ids that come from elsewhere (the rows another GPU sent): chunk c holds entries
// [c * chunk_len, (c + 1) * chunk_len) of ids.
static __global__ void __launch_bounds__(256) k_chunk_hist(const int32_t *__restrict__ ids, uint32_t A, uint32_t chunk_len,
                                                   uint32_t NE, uint32_t first_expert, uint32_t *__restrict__ chunk_hist) {
  __shared__ uint32_t hist[512];
  for (uint32_t i = threadIdx.x; i < NE; i += blockDim.x) hist[i] = 0;
  __syncthreads();
  const uint32_t a0 = blockIdx.x * chunk_len, a1 = min(A, a0 + chunk_len);
  for (uint32_t a = a0 + threadIdx.x; a < a1; a += blockDim.x) {
    const uint32_t e = (uint32_t)ids[a] - first_expert;
    if (e < NE) atomicAdd(&hist[e], 1u);
  }
  __syncthreads();
  for (uint32_t i = threadIdx.x; i < NE; i += blockDim.x) chunk_hist[(uint64_t)blockIdx.x * NE + i] = hist[i];
}

// The expert of every row a GPU receives in the rows' all-to-all: the sources one after another, each source's rows in
// expert order. cnt_all [world][NE] is every GPU's rows per expert; this GPU owns experts first .. first + per. Block
// b = source * per + local expert sums the runs before its own and fills its run.
static __global__ void __launch_bounds__(128) k_received_ids(const uint32_t *__restrict__ cnt_all, uint32_t NE, uint32_t first, uint32_t per,
                                                     int32_t *__restrict__ ids) {
  __shared__ uint32_t part[128];
  const uint32_t b = blockIdx.x;
  uint32_t sum = 0;
  for (uint32_t p = threadIdx.x; p < b; p += 128) sum += cnt_all[(uint64_t)(p / per) * NE + first + p % per];
  part[threadIdx.x] = sum;
  __syncthreads();
  for (uint32_t off = 64; off; off >>= 1) {
    if (threadIdx.x < off) part[threadIdx.x] += part[threadIdx.x + off];
    __syncthreads();
  }
  const uint32_t start = part[0], n = cnt_all[(uint64_t)(b / per) * NE + first + b % per];
  for (uint32_t i = threadIdx.x; i < n; i += 128) ids[start + i] = (int32_t)(first + b % per);
}

// dst[r] = src[row_src[r]] for r < R: the rows' f16 activations put in expert order, 16 bytes a thread, so that the
// tile kernels' bulk-tensor copies find a tile's rows one after another.
static __global__ void __launch_bounds__(256) k_gather_f16(const __half *__restrict__ src, const uint32_t *__restrict__ row_src, uint64_t R,
                                                   uint32_t K, __half *__restrict__ dst) {
  const uint64_t i = (uint64_t)blockIdx.x * 256 + threadIdx.x, per = K / 8, r = i / per;
  if (r >= R) return;
  const uint32_t c = (uint32_t)(i % per);
  ((uint4 *)(dst + r * K))[c] = __ldg((const uint4 *)(src + (uint64_t)row_src[r] * K) + c);
}

// ---------------------------------------------------------------------------------------------------------------
// Pack. Assignments a = t * K + k go into expert order by a stable counting sort: experts ascending, and inside an
// expert's run ascending a. The reference's fill takes rows by atomic increments, so its order inside a run depends on
// scheduling (prompt.cl:730-737); this one has no atomics on the order and gives the same permutation every time.

struct PackOut {
  uint32_t *cnt, *base;    // NE each
  uint32_t *chunk_off;     // [chunks][NE]: rows of the expert's run taken by earlier chunks
  MoeTile *tiles;          // expert order, <= 64 rows each (prompt.cl:719-723)
  MoeGroup *groups;        // <= group_max rows each: the experts with fewer than tensor_min rows
  BigTile *big;            // <= kTileN rows each: the others, for the tensor-core kernels
  uint32_t *counters;      // [0] tiles, [1] groups, [2] experts hit, [3] rows, [4] big tiles, [5] their rows
};

// Whether an expert with n rows goes to the tensor-core kernels (tensor_min 0: none does).
__host__ __device__ inline bool n_is_tensor(uint32_t n, uint32_t tensor_min) { return tensor_min != 0 && n >= tensor_min; }

// One CTA of 512 threads, thread e for expert e: sums the chunks' counts, scans them over the experts, writes tiles
// and groups. first_expert: the id of slot 0. group_max: the most rows a group holds (<= kGroupMax). tensor_budget, when
// not 0, lets the step lower tensor_min itself: to the least of 1, 2, 4, 8 rows that sends at most tensor_budget experts
// to the tile kernels. With skewed routing a short step has a few experts with many rows, which the tile kernels take
// in the time the integer-dot kernel needs for one of them; with even routing it has hundreds of experts with one or
// two rows, whose tiles would be all decode and no product: the threshold moves only if the experts that then change
// kernels hold at least half of the step's rows.
// The scan itself, for every thread of a CTA of 512 threads or more (the threads past 511 only keep the barriers):
// thread e < NE brings its expert's row count `run`; returns the first row of the expert's run.
__device__ __forceinline__ uint32_t pack_scan_block(uint32_t e, uint32_t run, uint32_t NE, uint32_t first_expert, uint32_t tensor_min,
                                                    uint32_t tensor_budget, uint32_t group_max, const PackOut &o) {
  __shared__ uint32_t s_rows[512], s_tiles[512], s_groups[512], s_hit[512], s_big[512], s_bigrows[512], s_hit2[512];
  __shared__ uint32_t s_rows_ge[3], s_total;
  const bool in = e < 512;
  if (!in || e >= NE) run = 0;
  if (tensor_budget) {
    // Lower only if the experts that would move hold at least half of the step's rows: moving a few rows costs two
    // more kernels for nothing.
    if (e < 3) s_rows_ge[e] = 0;
    if (e == 3) s_total = 0;
    __syncthreads();
    if (run >= 2) atomicAdd(&s_rows_ge[0], run);
    if (run >= 4) atomicAdd(&s_rows_ge[1], run);
    if (run >= 8) atomicAdd(&s_rows_ge[2], run);
    if (run) atomicAdd(&s_total, run);
    const uint32_t ge1 = __syncthreads_count(run >= 1), ge2 = __syncthreads_count(run >= 2), ge4 = __syncthreads_count(run >= 4),
                   ge8 = __syncthreads_count(run >= 8);
    if (ge1 <= tensor_budget) {
      tensor_min = 1;  // few experts in all: every one to the tile kernels
    } else {
      const int pick = ge2 <= tensor_budget ? 0 : ge4 <= tensor_budget ? 1 : ge8 <= tensor_budget ? 2 : -1;
      if (pick >= 0 && 2 * s_rows_ge[pick] >= s_total) tensor_min = min(tensor_min, 2u << pick);
    }
  }
  const bool tensor = n_is_tensor(run, tensor_min);
  const uint32_t n = run, nt = (n + kTileRows - 1) / kTileRows, ng = tensor ? 0 : (n + group_max - 1) / group_max;
  const uint32_t nb = tensor ? (n + kTileN - 1) / kTileN : 0;
  if (in) s_rows[e] = n, s_tiles[e] = nt, s_groups[e] = ng, s_hit[e] = n > 0, s_big[e] = nb, s_bigrows[e] = tensor ? n : 0;
  __syncthreads();
  for (uint32_t off = 1; off < 512; off <<= 1) {
    const bool take = in && e >= off;
    const uint32_t a = take ? s_rows[e - off] : 0, b = take ? s_tiles[e - off] : 0;
    const uint32_t c = take ? s_groups[e - off] : 0, d = take ? s_hit[e - off] : 0;
    const uint32_t f = take ? s_big[e - off] : 0, g = take ? s_bigrows[e - off] : 0;
    __syncthreads();
    if (in) s_rows[e] += a, s_tiles[e] += b, s_groups[e] += c, s_hit[e] += d, s_big[e] += f, s_bigrows[e] += g;
    __syncthreads();
  }
  const uint32_t first = in ? s_rows[e] - n : 0;
  if (e < NE) {
    o.cnt[e] = n;
    o.base[e] = first;
    const uint32_t tile0 = s_tiles[e] - nt, group0 = s_groups[e] - ng;
    for (uint32_t i = 0; i < nt; i++)
      o.tiles[tile0 + i] = MoeTile{first_expert + e, e, first + i * kTileRows, min(kTileRows, n - i * kTileRows)};
    for (uint32_t i = 0; i < ng; i++)
      o.groups[group0 + i] = MoeGroup{e, first + i * group_max, min(group_max, n - i * group_max)};
  }
  // Big tiles, sorted by size for the tile kernels' round-robin over CTAs: every full tile of kTileN rows first (in
  // expert order), then the experts' last, shorter tiles by falling row count (ties in expert order). s_bigrows is free
  // to reuse: the scan's total is read first.
  const uint32_t total_rows_big = s_bigrows[511], nfull = tensor ? n / kTileN : 0, rem = tensor ? n % kTileN : 0;
  __syncthreads();
  if (in) s_hit2[e] = nfull, s_bigrows[e] = rem;
  __syncthreads();
  for (uint32_t off = 1; off < 512; off <<= 1) {
    const uint32_t a = in && e >= off ? s_hit2[e - off] : 0;
    __syncthreads();
    if (in) s_hit2[e] += a;
    __syncthreads();
  }
  if (e < NE) {
    const uint32_t full0 = s_hit2[e] - nfull, all_full = s_hit2[511];
    for (uint32_t i = 0; i < nfull; i++) o.big[full0 + i] = BigTile{e, first + i * kTileN, kTileN};
    if (rem) {
      uint32_t rank = 0;
      for (uint32_t j = 0; j < 512; j++) rank += s_bigrows[j] > rem || (s_bigrows[j] == rem && j < e);
      o.big[all_full + rank] = BigTile{e, first + nfull * kTileN, rem};
    }
  }
  if (e == 511) {
    o.counters[0] = s_tiles[e], o.counters[1] = s_groups[e], o.counters[2] = s_hit[e], o.counters[3] = s_rows[e];
    o.counters[4] = s_big[e], o.counters[5] = total_rows_big;
  }
  return first;
}

static __global__ void __launch_bounds__(512) k_pack_scan(const uint32_t *__restrict__ chunk_hist, uint32_t nchunks, uint32_t NE,
                                                  uint32_t first_expert, uint32_t tensor_min, uint32_t tensor_budget, uint32_t group_max,
                                                  PackOut o) {
  const uint32_t e = threadIdx.x;
  uint32_t run = 0;
  if (e < NE) {
    // Sixteen chunks' counts are loaded at once: a lone CTA walking a thousand chunks one load at a time would spend
    // the stage on memory latency.
    for (uint32_t c0 = 0; c0 < nchunks; c0 += 16) {
      uint32_t v[16];
#pragma unroll
      for (uint32_t j = 0; j < 16; j++) v[j] = c0 + j < nchunks ? chunk_hist[(uint64_t)(c0 + j) * NE + e] : 0;
#pragma unroll
      for (uint32_t j = 0; j < 16; j++) {
        if (c0 + j < nchunks) o.chunk_off[(uint64_t)(c0 + j) * NE + e] = run;
        run += v[j];
      }
    }
  }
  pack_scan_block(e, run, NE, first_expert, tensor_min, tensor_budget, group_max, o);
}

// One CTA per chunk, thread e for expert e: walks the chunk's ids in order and hands out its expert's rows in that
// order. inv[a] = row; row_src[row] = a / src_div (the activation row the assignment reads: its token).
static __global__ void __launch_bounds__(512) k_pack_fill(const int32_t *__restrict__ ids, uint32_t A, uint32_t chunk_len, uint32_t NE,
                                                  const uint32_t *__restrict__ base, const uint32_t *__restrict__ chunk_off,
                                                  uint32_t src_div, uint32_t *__restrict__ inv, uint32_t *__restrict__ row_src,
                                                  uint32_t first_expert = 0) {
  extern __shared__ int32_t s_ids[];
  const uint32_t a0 = blockIdx.x * chunk_len, n = min(A, a0 + chunk_len) - a0;
  for (uint32_t i = threadIdx.x; i < n; i += blockDim.x) s_ids[i] = ids[a0 + i];
  __syncthreads();
  const uint32_t e = threadIdx.x;
  if (e >= NE) return;
  uint32_t row = base[e] + chunk_off[(uint64_t)blockIdx.x * NE + e];
  for (uint32_t i = 0; i < n; i++)
    if ((uint32_t)s_ids[i] - first_expert == e) {
      inv[a0 + i] = row;
      row_src[row] = (a0 + i) / src_div;
      row++;
    }
}

// A step of one chunk (at most kChunkTokens rows): top-k, scan and fill in one CTA, three launches less for the steps
// that launches bound. Dynamic shared memory kChunkTokens * K words for the chunk's ids.
static __global__ void __launch_bounds__(32 * kChunkTokens, 1) k_router_topk_pack(const float *__restrict__ rl, const float *__restrict__ bias, uint32_t T,
                                                                       uint32_t NE, uint32_t K, int32_t *__restrict__ ids, float *__restrict__ w,
                                                                       float *__restrict__ gs, uint32_t tensor_min, uint32_t tensor_budget,
                                                                       uint32_t group_max, PackOut o, uint32_t *__restrict__ inv,
                                                                       uint32_t *__restrict__ row_src) {
  __shared__ uint32_t hist[512];
  extern __shared__ int32_t s_chunk_ids[];
  router_topk_block(rl, nullptr, bias, nullptr, 0, T, NE, K, ids, w, gs, hist, s_chunk_ids);
  const uint32_t e = threadIdx.x;
  const uint32_t run = e < NE ? hist[e] : 0;
  uint32_t row = pack_scan_block(e, run, NE, 0, tensor_min, tensor_budget, group_max, o);
  if (e < NE && run) {
    const uint32_t A = T * K;
    for (uint32_t i = 0; i < A; i++)
      if ((uint32_t)s_chunk_ids[i] == e) {
        inv[i] = row;
        row_src[row] = i / K;
        row++;
      }
  }
}

// ---------------------------------------------------------------------------------------------------------------
// Combine: out[t] = sum over k, in rank order, of w[t][k] * y[inv[t K + k]] + gs[t] * s[t], in f32 (layer.cl:874-877).
// One CTA per row. y is f32, or f16 when it came back from other GPUs in that form.
__device__ __forceinline__ float4 load_row4(const float *y, uint64_t row, uint32_t E, uint32_t i) { return ((const float4 *)(y + row * E))[i]; }
__device__ __forceinline__ float4 load_row4(const __half *y, uint64_t row, uint32_t E, uint32_t i) {
  const uint2 u = ((const uint2 *)(y + row * E))[i];
  const float2 a = __half22float2(*(const __half2 *)&u.x), b = __half22float2(*(const __half2 *)&u.y);
  return make_float4(a.x, a.y, b.x, b.y);
}
template <class Y>
static __global__ void __launch_bounds__(256) k_combine(const Y *__restrict__ y, const uint32_t *__restrict__ inv,
                                                       const float *__restrict__ w, const float *__restrict__ gs,
                                                       const float *__restrict__ s, uint32_t K, uint32_t E, float *__restrict__ out) {
  const uint32_t t = blockIdx.x;
  __shared__ uint32_t rows[16];
  __shared__ float wk[16];
  if (threadIdx.x < K) rows[threadIdx.x] = inv[(uint64_t)t * K + threadIdx.x], wk[threadIdx.x] = w[(uint64_t)t * K + threadIdx.x];
  __syncthreads();
  const float g = s ? gs[t] : 0.0f;
  for (uint32_t i = threadIdx.x; i < E / 4; i += 256) {
    float4 acc = make_float4(0, 0, 0, 0);
    for (uint32_t k = 0; k < K; k++) {
      const float4 v = load_row4(y, rows[k], E, i);
      acc.x = fmaf(wk[k], v.x, acc.x), acc.y = fmaf(wk[k], v.y, acc.y);
      acc.z = fmaf(wk[k], v.z, acc.z), acc.w = fmaf(wk[k], v.w, acc.w);
    }
    if (s) {
      const float4 v = ((const float4 *)(s + (uint64_t)t * E))[i];
      acc.x = fmaf(g, v.x, acc.x), acc.y = fmaf(g, v.y, acc.y), acc.z = fmaf(g, v.z, acc.z), acc.w = fmaf(g, v.w, acc.w);
    }
    ((float4 *)(out + (uint64_t)t * E))[i] = acc;
  }
}

// ---------------------------------------------------------------------------------------------------------------
// Expert parallel: the rows that cross GPUs. A wire row is one quantised activation row packed: K codes, its scales,
// q8_K's sums, padded to 16 bytes.
__host__ __device__ constexpr uint32_t wire_row_bytes(bool q8k, uint32_t K) { return (K + (q8k ? K / 64 + K / 8 : K / 8) + 15) & ~15u; }

// wire[r] = the quantised row of the token assignment row r reads (row_src[r]); ids_sorted[r] = its expert. One warp
// per row.
static __global__ void __launch_bounds__(256) k_gather_wire(const ActView act, uint32_t K, bool q8k, const uint32_t *__restrict__ row_src,
                                                           const uint32_t *__restrict__ inv, const int32_t *__restrict__ ids, uint32_t A,
                                                           uint8_t *__restrict__ wire, int32_t *__restrict__ ids_sorted) {
  const uint32_t lane = threadIdx.x % 32;
  const uint64_t r = (uint64_t)blockIdx.x * 8 + threadIdx.x / 32;
  if (r >= A) return;
  const uint32_t wb = wire_row_bytes(q8k, K), t = row_src[r], dbytes = q8k ? K / 64 : K / 8;
  uint8_t *dst = wire + r * wb;
  const int4 *q = (const int4 *)(act.q + (uint64_t)t * act.q_stride);
  for (uint32_t i = lane; i < K / 16; i += 32) ((int4 *)dst)[i] = q[i];
  const uint32_t *d = (const uint32_t *)((const uint8_t *)act.d + (uint64_t)t * act.d_stride);
  for (uint32_t i = lane; i < dbytes / 4; i += 32) ((uint32_t *)(dst + K))[i] = d[i];
  if (q8k) {
    const uint32_t *b = (const uint32_t *)((const uint8_t *)act.bs + (uint64_t)t * act.bs_stride);
    for (uint32_t i = lane; i < K / 32; i += 32) ((uint32_t *)(dst + K + dbytes))[i] = b[i];
  }
  // The ids in expert order: assignment a sits at row inv[a]. Here r also counts the assignments.
  if (lane == 0) ids_sorted[inv[r]] = ids[r];
}

// The f16 operand of the tensor-core kernels from wire rows: code * scale, as the quantisers write it. One warp per
// 256 values.
static __global__ void __launch_bounds__(256) k_wire_to_f16(const uint8_t *__restrict__ wire, uint32_t K, bool q8k, uint64_t nblk256,
                                                           __half *__restrict__ out) {
  const uint64_t blk = (uint64_t)blockIdx.x * 8 + threadIdx.x / 32;
  if (blk >= nblk256) return;
  const uint32_t lane = threadIdx.x % 32, per_row = K / 256, wb = wire_row_bytes(q8k, K);
  const uint64_t row = blk / per_row;
  const uint32_t b = (uint32_t)(blk % per_row);
  const uint8_t *src = wire + row * wb;
  const char4 lo = ((const char4 *)(src + 256 * b))[2 * lane], hi = ((const char4 *)(src + 256 * b))[2 * lane + 1];
  const float d = q8k ? ((const float *)(src + K))[b] : ((const float *)(src + K))[8 * b + lane / 4];
  const __half2 h0 = __floats2half2_rn(d * (float)lo.x, d * (float)lo.y), h1 = __floats2half2_rn(d * (float)lo.z, d * (float)lo.w);
  const __half2 h2 = __floats2half2_rn(d * (float)hi.x, d * (float)hi.y), h3 = __floats2half2_rn(d * (float)hi.z, d * (float)hi.w);
  uint4 o;
  o.x = *(const uint32_t *)&h0, o.y = *(const uint32_t *)&h1, o.z = *(const uint32_t *)&h2, o.w = *(const uint32_t *)&h3;
  ((uint4 *)(out + row * K + 256 * b))[lane] = o;
}

// out[r] = y[inv[r]]: the experts' rows back in the order they arrived, as f32 or f16. One CTA per row.
template <class O>
static __global__ void __launch_bounds__(256) k_unpermute(const float *__restrict__ y, const uint32_t *__restrict__ inv, uint32_t E,
                                                         O *__restrict__ out) {
  const uint64_t r = blockIdx.x;
  const float4 *src = (const float4 *)(y + (uint64_t)inv[r] * E);
  for (uint32_t i = threadIdx.x; i < E / 4; i += 256) {
    const float4 v = src[i];
    if constexpr (sizeof(O) == 4) {
      ((float4 *)(out + r * E))[i] = v;
    } else {
      const __half2 a = __floats2half2_rn(v.x, v.y), b = __floats2half2_rn(v.z, v.w);
      uint2 o;
      o.x = *(const uint32_t *)&a, o.y = *(const uint32_t *)&b;
      ((uint2 *)(out + r * E))[i] = o;
    }
  }
}

}  // namespace moe
