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

// What the tensor-core router product takes of a row (steps of many rows): x as the sum of two f16 numbers, hi = f16(x)
// and lo = f16(x - hi), 22 bits of x between them, and the block's sum of squares, from which the top-k kernel bounds
// that product's error for the row.
struct RouterSplit {
  __half *hi, *lo;     // [rows][K] each; null: not wanted
  float *norm2_parts;  // [rows][K / 256]
};
__device__ __forceinline__ uint32_t split_pair(float x0, float x1, uint32_t &lo) {
  const __half2 h = __floats2half2_rn(x0, x1);
  const float2 hf = __half22float2(h);
  const __half2 l = __floats2half2_rn(x0 - hf.x, x1 - hf.y);
  lo = *(const uint32_t *)&l;
  return *(const uint32_t *)&h;
}
__device__ __forceinline__ void router_split(const float4 &a, const float4 &b, uint64_t blk, uint32_t lane, const RouterSplit &rs) {
  uint4 hi, lo;
  hi.x = split_pair(a.x, a.y, lo.x), hi.y = split_pair(a.z, a.w, lo.y);
  hi.z = split_pair(b.x, b.y, lo.z), hi.w = split_pair(b.z, b.w, lo.w);
  ((uint4 *)(rs.hi + blk * 256))[lane] = hi;
  ((uint4 *)(rs.lo + blk * 256))[lane] = lo;
  float s = a.x * a.x + a.y * a.y + a.z * a.z + a.w * a.w + b.x * b.x + b.y * b.y + b.z * b.z + b.w * b.w;
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
  if (lane == 0) rs.norm2_parts[blk] = s;
}

static __global__ void __launch_bounds__(256) k_quant_q8_0(const float *__restrict__ x, uint64_t nblk256, int8_t *__restrict__ q,
                                                   float *__restrict__ d, __half *__restrict__ deq, const float *__restrict__ gate,
                                                   uint32_t per_row, float *__restrict__ gate_parts, RouterSplit rs) {
  dependents_may_launch(), wait_for_predecessors();
  const uint64_t blk = (uint64_t)blockIdx.x * 8 + threadIdx.x / 32;
  if (blk >= nblk256) return;
  const uint32_t lane = threadIdx.x % 32;
  const float4 a = ((const float4 *)(x + blk * 256))[2 * lane], b = ((const float4 *)(x + blk * 256))[2 * lane + 1];
  if (gate) gate_part(a, b, gate, per_row, blk, lane, gate_parts);
  if (rs.hi) router_split(a, b, blk, lane, rs);
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
                                                   const float *__restrict__ gate, uint32_t per_row, float *__restrict__ gate_parts,
                                                   RouterSplit rs) {
  dependents_may_launch(), wait_for_predecessors();
  const uint64_t blk = (uint64_t)blockIdx.x * 8 + threadIdx.x / 32;
  if (blk >= nblk256) return;
  const uint32_t lane = threadIdx.x % 32;
  const float4 a = ((const float4 *)(x + blk * 256))[2 * lane], b = ((const float4 *)(x + blk * 256))[2 * lane + 1];
  if (gate) gate_part(a, b, gate, per_row, blk, lane, gate_parts);
  if (rs.hi) router_split(a, b, blk, lane, rs);
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

// Steps of many rows: the logits come from the tensor-core product (router_mma.cuh) and are approximate. For row t
// every one is within eps_t of the logit the exact order gives, eps_t = eps_rel * |x_t| * (largest |w_e|) + eps_abs,
// with |x_t|^2 summed from norm2_parts. The top-k below then recomputes, in the exact order, only what that bound
// cannot decide.
struct RouterApprox {
  const float *logits;       // [T][NE]; null: the logits are exact rows rl[t][NE + 1]
  const float *x;            // [T][E]
  const float *W;            // [NE][E]
  const float *norm2_parts;  // [T][nparts]
  const float *gate_parts;   // [T][nparts]: the parts of the shared expert's gate logit
  uint32_t E, nparts;
  float eps_rel, eps_abs;
};

// The logits of up to four experts for row x, each exactly as k_router_logits_rows and the CPU oracle sum it: eight
// pieces of the row, each a chain of fused multiply-adds from 0 in index order, the pieces added in order, the bias
// last. Lane 8 j + s takes piece s of expert ex[j]; lanes 8 j .. 8 j + 7 return expert ex[j]'s logit.
__device__ __forceinline__ float exact_logits4(const float *__restrict__ x, const float *__restrict__ W, const float *__restrict__ bias,
                                               uint32_t E, uint32_t e, uint32_t lane) {
  const uint32_t piece = E / kRouterPieces, s = lane % 8;
  const float4 *xp = (const float4 *)(x + s * piece), *wp = (const float4 *)(W + (uint64_t)e * E + s * piece);
  float p = 0.0f;
  // Eight loads of each operand in flight a lane: the chain of multiply-adds is short beside a trip to memory, so the
  // pass costs about piece / 32 such trips.
  for (uint32_t i = 0; i < piece / 4; i += 8) {
    float4 xv[8], wv[8];
#pragma unroll
    for (int j = 0; j < 8; j++) xv[j] = __ldg(xp + i + j), wv[j] = __ldg(wp + i + j);
#pragma unroll
    for (int j = 0; j < 8; j++) {
      p = fmaf(xv[j].x, wv[j].x, p);
      p = fmaf(xv[j].y, wv[j].y, p);
      p = fmaf(xv[j].z, wv[j].z, p);
      p = fmaf(xv[j].w, wv[j].w, p);
    }
  }
  float tot = __shfl_sync(0xffffffffu, p, lane & ~7u);
#pragma unroll
  for (int j = 1; j < (int)kRouterPieces; j++) tot = __fadd_rn(tot, __shfl_sync(0xffffffffu, p, (lane & ~7u) + j));
  if (bias) tot = __fadd_rn(tot, bias[e]);
  return tot;
}

// exact_logits4 with the operands brought through shared memory. A lane walking its own piece of a row from global
// memory touches, with the other lanes, 32 different lines an instruction, and the tag stage of L1 then sets the pace
// (measured: two thirds of its peak, the kernel's limit). Here the warp copies the row and the four experts' rows
// chunk by chunk with 16-byte asynchronous copies, eight lanes to a piece's 128 contiguous bytes, the next chunk on
// its way while this one is summed; the lanes read their pieces from shared memory, whose padding (a piece's chunk
// every 144 bytes) spreads a quarter-warp's eight 16-byte reads over all banks. The sums are the same chains.
constexpr uint32_t kExChunk = 32;                        // values of each piece a chunk holds
constexpr uint32_t kExPiece = kExChunk * 4 + 16;         // bytes from one piece's chunk to the next in shared memory
constexpr uint32_t kExRow = kRouterPieces * kExPiece;    // a row's chunk: 1,152 bytes
constexpr uint32_t kExBuf = 5 * kExRow;                  // the row and four experts' rows
constexpr uint32_t kExWarpBytes = 2 * kExBuf;            // two chunks: 11,520 bytes a warp
__device__ __forceinline__ void cp_async16(uint32_t dst_smem, const void *src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst_smem), "l"(src) : "memory");
}
__device__ __forceinline__ float exact_logits4_staged(const float *__restrict__ x, const float *__restrict__ W, const float *__restrict__ bias,
                                                      uint32_t E, uint32_t e, uint32_t lane, uint8_t *buf) {
  const uint32_t piece = E / kRouterPieces, nch = piece / kExChunk, s = lane % 8, g = lane / 8;
  const uint32_t buf32 = (uint32_t)__cvta_generic_to_shared(buf);
  // The four experts of the pass, known to every lane.
  uint32_t ex[4];
#pragma unroll
  for (int j = 0; j < 4; j++) ex[j] = __shfl_sync(0xffffffffu, e, 8 * j);
  auto issue = [&](uint32_t c, uint32_t b) {
    // A row's chunk is 8 pieces x 128 bytes: 64 copies of 16 bytes, two a lane.
#pragma unroll
    for (int k = 0; k < 2; k++) {
      const uint32_t idx = k * 32 + lane, pc = idx / 8, j = idx % 8;
      const uint64_t off = (uint64_t)pc * piece + c * kExChunk + j * 4;
      const uint32_t dst = buf32 + b * kExBuf + pc * kExPiece + j * 16;
      cp_async16(dst, x + off);
#pragma unroll
      for (int r = 0; r < 4; r++) cp_async16(dst + (1 + r) * kExRow, W + (uint64_t)ex[r] * E + off);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  float p = 0.0f;
  issue(0, 0);
  for (uint32_t c = 0; c < nch; c++) {
    if (c + 1 < nch) {
      issue(c + 1, (c + 1) & 1);
      asm volatile("cp.async.wait_group 1;" ::: "memory");
    } else {
      asm volatile("cp.async.wait_group 0;" ::: "memory");
    }
    __syncwarp();
    const float4 *xs = (const float4 *)(buf + (c & 1) * kExBuf + s * kExPiece);
    const float4 *ws = (const float4 *)(buf + (c & 1) * kExBuf + (1 + g) * kExRow + s * kExPiece);
#pragma unroll
    for (int j = 0; j < (int)kExChunk / 4; j++) {
      const float4 xv = xs[j], wv = ws[j];
      p = fmaf(xv.x, wv.x, p);
      p = fmaf(xv.y, wv.y, p);
      p = fmaf(xv.z, wv.z, p);
      p = fmaf(xv.w, wv.w, p);
    }
    __syncwarp();  // every lane has read the chunk before its buffer is filled again
  }
  float tot = __shfl_sync(0xffffffffu, p, lane & ~7u);
#pragma unroll
  for (int j = 1; j < (int)kRouterPieces; j++) tot = __fadd_rn(tot, __shfl_sync(0xffffffffu, p, (lane & ~7u) + j));
  if (bias) tot = __fadd_rn(tot, bias[e]);
  return tot;
}

// The block's part: its rows' ids, weights and gates written, the chunk's count of every expert left in hist (shared,
// 512 words) and, when s_ids is not null, the chunk's ids there too (shared, kChunkTokens * K words).
//
// With approximate logits a row's candidates are the experts whose approximate logit is within 2 eps of the K-th
// largest: the true top K is among them (an expert outside is below K others by more than the two errors can
// bridge). Sorted by approximate logit, two neighbours less than 2 eps apart cannot be ordered by it, and both get
// their exact logit; any other pair's order is certain. The candidates are then ranked by (logit, lower expert first)
// with exact logits where they were needed, and the first K are the row's experts, in rank order. A row with more
// than 32 candidates (all logits equal, as for a row of zeros) or a logit that is not finite (an x beyond f16's range)
// has every logit recomputed exactly instead.
__device__ __forceinline__ void router_topk_block(const float *__restrict__ rl, const RouterApprox ap, const float *__restrict__ bias,
                                                  uint32_t T, uint32_t NE, uint32_t K, int32_t *__restrict__ ids, float *__restrict__ w,
                                                  float *__restrict__ gs, uint32_t *hist, int32_t *s_ids, uint8_t *ex_smem = nullptr) {
  // hist null: the caller counts the chunks' experts itself (k_chunk_hist), and the block may be of any number of warps.
  // ex_smem: kExWarpBytes of shared memory for every warp of the block, through which the exact sums then take their
  // operands (E a multiple of 8 * kExChunk); null: straight from global memory.
  uint8_t *ex_buf = ex_smem ? ex_smem + (threadIdx.x / 32) * kExWarpBytes : nullptr;
  auto exact4 = [&](const float *xr, uint32_t e, uint32_t ln) {
    return ex_buf ? exact_logits4_staged(xr, ap.W, bias, ap.E, e, ln, ex_buf) : exact_logits4(xr, ap.W, bias, ap.E, e, ln);
  };
  if (hist) {
    for (uint32_t i = threadIdx.x; i < NE; i += blockDim.x) hist[i] = 0;
    __syncthreads();
  }
  const uint32_t lane = threadIdx.x % 32, t = blockIdx.x * (blockDim.x / 32) + threadIdx.x / 32, per = NE / 32;
  if (t < T) {
    uint32_t key[kMaxPerLane];
    float mx = -INFINITY, eps2 = 0.0f;  // eps2: twice the row's error bound; 0 with exact logits
    bool finite = true;
    if (ap.logits) {
      // The row itself is wanted only if some logits have to be recomputed, but then at once: ask for it now.
      const char *row = (const char *)(ap.x + (uint64_t)t * ap.E);
      for (uint32_t b = lane * 128; b < ap.E * 4; b += 32 * 128) asm volatile("prefetch.global.L2 [%0];" ::"l"(row + b));
    }
#pragma unroll
    for (int j = 0; j < kMaxPerLane; j++) {
      key[j] = 0;
      if ((uint32_t)j < per) {
        const uint32_t e = lane + 32 * j;
        float f;
        if (ap.logits) {
          f = ap.logits[(uint64_t)t * NE + e];
          if (bias) f = __fadd_rn(f, bias[e]);
          finite = finite && isfinite(f);
        } else {
          f = rl[(uint64_t)t * (NE + 1) + e];
        }
        key[j] = order_key(f);
        mx = fmaxf(mx, f);
      }
    }
    if (ap.logits) {
      float n2 = 0.0f;
      for (uint32_t p = lane; p < ap.nparts; p += 32) n2 += ap.norm2_parts[(uint64_t)t * ap.nparts + p];
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) n2 += __shfl_xor_sync(0xffffffffu, n2, off);
      eps2 = 2.0f * (ap.eps_rel * sqrtf(n2) + ap.eps_abs);
      finite = __all_sync(0xffffffffu, finite) && isfinite(eps2);
    }
    // Lane k keeps the k-th winner of the rounds below.
    float my_v = 0.0f, sum = 0.0f;
    uint32_t my_id = 0, ncand = 0;
    for (bool exact_all = ap.logits && !finite;;) {
      if (exact_all) {
        // Every logit exactly, four experts a pass: for rows the approximate ones cannot serve.
        mx = -INFINITY;
        for (uint32_t e0 = 0; e0 < NE; e0 += 4) {
          const float v = exact4(ap.x + (uint64_t)t * ap.E, e0 + lane / 8, lane);
#pragma unroll
          for (int q = 0; q < 4; q++) {
            const float vq = __shfl_sync(0xffffffffu, v, 8 * q);
            const uint32_t e = e0 + q;
            if (e % 32 == lane) {
#pragma unroll
              for (int j = 0; j < kMaxPerLane; j++)
                if ((uint32_t)j == e / 32) key[j] = order_key(vq);
            }
            mx = fmaxf(mx, vq);
          }
        }
        eps2 = 0.0f;
      }
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
      sum = 0.0f;
#pragma unroll
      for (int j = 0; j < kMaxPerLane; j++)
        if ((uint32_t)j < per) sum += expf(key_value(key[j]) - mx);
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
      // Rounds of arg-max over (key, lower expert first), which use the keys up. K rounds with exact logits; with
      // approximate ones, on until the next is more than 2 eps below the K-th (at most 32 in all).
      float vK = 0.0f;
      bool overflow = false;
      ncand = 0;
      // A lane keeps the best of its own keys (the lower expert among equals); a round is then two warp reductions,
      // the largest key and among its holders the lowest expert, and only the winner's lane has a new best to find.
      uint32_t lkey = 0, lj = 0;
      auto rescan = [&]() {
        lkey = 0, lj = 0;
#pragma unroll
        for (int j = 0; j < kMaxPerLane; j++)
          if ((uint32_t)j < per && key[j] > lkey) lkey = key[j], lj = j;
      };
      rescan();
      for (uint32_t k = 0; k < 32; k++) {
        const uint32_t bkey = __reduce_max_sync(0xffffffffu, lkey);
        if (bkey == 0) break;  // nothing left (fewer than 32 experts in all)
        const uint32_t e = __reduce_min_sync(0xffffffffu, lkey == bkey ? lane + 32 * lj : 0xFFFFFFFFu);
        const float v = key_value(bkey);
        if (k == K - 1) vK = v;
        if (k >= K && !(eps2 > 0.0f && v >= vK - eps2)) break;
        if (e % 32 == lane) {
#pragma unroll
          for (int j = 0; j < kMaxPerLane; j++)
            if ((uint32_t)j == e / 32) key[j] = 0;
          rescan();
        }
        if (lane == k) my_id = e, my_v = v;
        ncand = k + 1;
        if (k == 31 && eps2 > 0.0f && NE > 32) overflow = true;  // there may be more within reach than a warp holds
      }
      if (!overflow) break;
      exact_all = true;
    }
    if (eps2 > 0.0f) {
      // Neighbours too close to order: both get their exact logit, four candidates a pass.
      const float up = __shfl_up_sync(0xffffffffu, my_v, 1), down = __shfl_down_sync(0xffffffffu, my_v, 1);
      const bool need = lane < ncand && ((lane > 0 && up - my_v <= eps2) || (lane + 1 < ncand && my_v - down <= eps2));
      uint32_t todo = __ballot_sync(0xffffffffu, need);
      while (todo) {
        uint32_t c[4];
#pragma unroll
        for (int q = 0; q < 4; q++) {
          c[q] = todo ? (uint32_t)__ffs(todo) - 1 : 0xFFFFFFFFu;
          if (todo) todo &= todo - 1;
        }
        const uint32_t g8 = lane / 8, mine = g8 == 0 ? c[0] : g8 == 1 ? c[1] : g8 == 2 ? c[2] : c[3];
        const uint32_t e = __shfl_sync(0xffffffffu, my_id, mine == 0xFFFFFFFFu ? 0 : mine);
        const float v = exact4(ap.x + (uint64_t)t * ap.E, e, lane);
#pragma unroll
        for (int q = 0; q < 4; q++) {
          const float vq = __shfl_sync(0xffffffffu, v, 8 * q);
          if (lane == c[q]) my_v = vq + 0.0f;
        }
      }
    }
    // Rank among the candidates by (logit, lower expert first); with exact logits this is the order they came in.
    uint32_t rank = 0;
    {
      const unsigned long long me = ((unsigned long long)order_key(my_v) << 32) | (uint32_t)~my_id;
      for (uint32_t j = 0; j < ncand; j++) {
        const unsigned long long o = __shfl_sync(0xffffffffu, me, j);
        rank += o > me;
      }
    }
    const bool winner = lane < ncand && rank < K;
    const float pk = winner ? expf(my_v - mx) / sum : 0.0f;
    // The K winners' p added in rank order.
    float tot = 0.0f;
    for (uint32_t k = 0; k < K; k++) {
      const uint32_t src = __ffs(__ballot_sync(0xffffffffu, winner && rank == k)) - 1;
      tot += __shfl_sync(0xffffffffu, pk, src & 31);
    }
    if (winner) {
      ids[(uint64_t)t * K + rank] = (int32_t)my_id;
      w[(uint64_t)t * K + rank] = pk / fmaxf(tot, 6.1035e-5f);
      if (hist) atomicAdd(&hist[my_id], 1u);
      if (s_ids) s_ids[(threadIdx.x / 32) * K + rank] = (int32_t)my_id;
    }
    if (lane == 0) {
      float g;
      if (ap.logits) {
        g = 0.0f;
        for (uint32_t p = 0; p < ap.nparts; p++) g += ap.gate_parts[(uint64_t)t * ap.nparts + p];
      } else {
        g = rl[(uint64_t)t * (NE + 1) + NE];
      }
      gs[t] = 1.0f / (1.0f + expf(-g));
    }
  }
  if (hist) __syncthreads();
}

// The top-k alone, a few rows a CTA and no barrier in it: for long steps, whose rows wait on memory for their exact
// recomputations; with many small CTAs an SM always has rows that are not waiting, and no row waits for the slowest of
// its chunk. The chunks' counts then come from k_chunk_hist.
constexpr uint32_t kTopkRowsPerCta = 4;
static __global__ void __launch_bounds__(32 * kTopkRowsPerCta) k_router_topk_rows(const RouterApprox ap, const float *__restrict__ bias, uint32_t T,
                                                                                 uint32_t NE, uint32_t K, int32_t *__restrict__ ids,
                                                                                 float *__restrict__ w, float *__restrict__ gs) {
  __shared__ __align__(16) uint8_t ex_smem[kTopkRowsPerCta * kExWarpBytes];
  router_topk_block(nullptr, ap, bias, T, NE, K, ids, w, gs, nullptr, nullptr, ap.E % (kRouterPieces * kExChunk) == 0 ? ex_smem : nullptr);
}

static __global__ void __launch_bounds__(32 * kChunkTokens) k_router_topk(const float *__restrict__ rl, const RouterApprox ap,
                                                                  const float *__restrict__ bias, uint32_t T, uint32_t NE,
                                                                  uint32_t K, int32_t *__restrict__ ids,
                                                                  float *__restrict__ w, float *__restrict__ gs,
                                                                  uint32_t *__restrict__ chunk_hist) {
  __shared__ uint32_t hist[512];
  router_topk_block(rl, ap, bias, T, NE, K, ids, w, gs, hist, nullptr);
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

// The rows' f16 activations put in expert order, so that the tile kernels' bulk-tensor copies find a tile's rows one
// after another (the reference's p_moe_scatter, kernels/models/qwen4exp/prompt.cl:744-754), for a step whose every row has
// `per_row` places in expert order, place_of[t * per_row + k]: dst[place_of[t * per_row + k]] = src[t]. A CTA a row; a
// thread reads 16 bytes of it once and writes them per_row times. (The same copy taken from the places' side, dst[r] =
// src[row_src[r]], reads a row once per place, in expert order, long after its last use left the L2: at 32,768 rows
// of 2,048 values and ten places a row it read 1.0 GB from DRAM for the 134 MB of rows there are, and took twice as long.)
static __global__ void __launch_bounds__(256) k_scatter_f16(const __half *__restrict__ src, const uint32_t *__restrict__ place_of, uint32_t per_row,
                                                    uint32_t K, __half *__restrict__ dst) {
  const uint64_t t = blockIdx.x;
  const uint32_t *places = place_of + t * per_row;
  for (uint32_t c = threadIdx.x; c < K / 8; c += 256) {
    const uint4 v = __ldg((const uint4 *)(src + t * K) + c);
    for (uint32_t k = 0; k < per_row; k++) ((uint4 *)(dst + (uint64_t)__ldg(places + k) * K))[c] = v;
  }
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
  // Big tiles, in the order the tile kernels deal them to their CTAs round by round. First the experts that have at
  // least one full tile of kTileN rows, in expert order, each one's tiles side by side, its last, shorter one too: the
  // CTAs that take them run at the same time, so an expert's weights come from HBM once and from L2 after that (with
  // the short tiles all at the end, as this list once had them, every expert's weights were read from HBM again for
  // its short tile: 3.5 GB of traffic a 32,768-row gate/up launch against 2.6 GB the algorithm needs). Then the experts
  // with one short tile only, by falling row count (ties in expert order), so that the last rounds hold the
  // shortest items. s_bigrows is free to reuse: the scan's total is read first.
  const uint32_t total_rows_big = s_bigrows[511], nfull = tensor ? n / kTileN : 0, rem = tensor ? n % kTileN : 0;
  const uint32_t mine = nfull ? nfull + (rem != 0) : 0;
  __syncthreads();
  if (in) s_hit2[e] = mine, s_bigrows[e] = nfull ? 0 : rem;
  __syncthreads();
  for (uint32_t off = 1; off < 512; off <<= 1) {
    const uint32_t a = in && e >= off ? s_hit2[e - off] : 0;
    __syncthreads();
    if (in) s_hit2[e] += a;
    __syncthreads();
  }
  if (e < NE) {
    const uint32_t tile0 = s_hit2[e] - mine, all_long = s_hit2[511];
    for (uint32_t i = 0; i < mine; i++) o.big[tile0 + i] = BigTile{e, first + i * kTileN, i < nfull ? kTileN : rem};
    if (!nfull && rem) {
      uint32_t rank = 0;
      for (uint32_t j = 0; j < 512; j++) rank += s_bigrows[j] > rem || (s_bigrows[j] == rem && j < e);
      o.big[all_long + rank] = BigTile{e, first, rem};
    }
  }
  if (e == 511) {
    o.counters[0] = s_tiles[e], o.counters[1] = s_groups[e], o.counters[2] = s_hit[e], o.counters[3] = s_rows[e];
    o.counters[4] = s_big[e], o.counters[5] = total_rows_big;
  }
  return first;
}

// The scan over a long step's chunks in two levels: a CTA per kScanGroup chunks leaves every expert's running count
// within its group in chunk_off and the group's total in group_tot; k_pack_scan then walks the groups' totals instead
// of the chunks, and k_pack_fill adds a chunk's group's offset to the chunk's own. (One CTA walking a thousand chunks
// took 133 us of a 32,768-row step.)
constexpr uint32_t kScanGroup = 32;
static __global__ void __launch_bounds__(512) k_pack_scan_groups(const uint32_t *__restrict__ chunk_hist, uint32_t nchunks, uint32_t NE,
                                                         uint32_t *__restrict__ chunk_off, uint32_t *__restrict__ group_tot) {
  const uint32_t e = threadIdx.x, c_begin = blockIdx.x * kScanGroup, c_end = min(nchunks, c_begin + kScanGroup);
  if (e >= NE) return;
  uint32_t run = 0;
  for (uint32_t c0 = c_begin; c0 < c_end; c0 += 16) {
    uint32_t v[16];
#pragma unroll
    for (uint32_t j = 0; j < 16; j++) v[j] = c0 + j < c_end ? chunk_hist[(uint64_t)(c0 + j) * NE + e] : 0;
#pragma unroll
    for (uint32_t j = 0; j < 16; j++) {
      if (c0 + j < c_end) chunk_off[(uint64_t)(c0 + j) * NE + e] = run;
      run += v[j];
    }
  }
  group_tot[(uint64_t)blockIdx.x * NE + e] = run;
}

// groups: null, or the groups' totals left by k_pack_scan_groups, [ngroups][NE], which become the groups' offsets in place.
static __global__ void __launch_bounds__(512) k_pack_scan(const uint32_t *__restrict__ chunk_hist, uint32_t nchunks, uint32_t NE,
                                                  uint32_t first_expert, uint32_t tensor_min, uint32_t tensor_budget, uint32_t group_max,
                                                  PackOut o, uint32_t *__restrict__ groups = nullptr, uint32_t ngroups = 0) {
  const uint32_t e = threadIdx.x;
  uint32_t run = 0;
  if (e < NE && groups) {
    for (uint32_t g0 = 0; g0 < ngroups; g0 += 16) {
      uint32_t v[16];
#pragma unroll
      for (uint32_t j = 0; j < 16; j++) v[j] = g0 + j < ngroups ? groups[(uint64_t)(g0 + j) * NE + e] : 0;
#pragma unroll
      for (uint32_t j = 0; j < 16; j++) {
        if (g0 + j < ngroups) groups[(uint64_t)(g0 + j) * NE + e] = run;
        run += v[j];
      }
    }
  } else if (e < NE) {
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

// One CTA per chunk: the chunk's entries take their expert's rows in the order they stand in.
// inv[a] = row; row_src[row] = a / src_div (the activation row the assignment reads: its token). Dynamic shared
// memory 16 * NE words.
static __global__ void __launch_bounds__(512) k_pack_fill(const int32_t *__restrict__ ids, uint32_t A, uint32_t chunk_len, uint32_t NE,
                                                  const uint32_t *__restrict__ base, const uint32_t *__restrict__ chunk_off,
                                                  uint32_t src_div, uint32_t *__restrict__ inv, uint32_t *__restrict__ row_src,
                                                  uint32_t first_expert = 0, const uint32_t *__restrict__ group_off = nullptr) {
  // A thread an entry (chunk_len <= 512). An entry's row is its expert's first row for this chunk plus the number of
  // the chunk's earlier entries with the same expert: those of earlier warps, counted per (warp, expert) in shared
  // memory and summed over the warps, and those of lower lanes of its own warp, which match_any names. (A thread an
  // expert, each walking the chunk's entries, took 52 us of a 32,768-row step.)
  extern __shared__ uint32_t s_cnt[];  // [16][NE]
  const uint32_t a0 = blockIdx.x * chunk_len, n = min(A, a0 + chunk_len) - a0;
  const uint32_t i = threadIdx.x, warp = i / 32, lane = i % 32;
  for (uint32_t k = i; k < 16 * NE; k += 512) s_cnt[k] = 0;
  const uint32_t e = i < n ? (uint32_t)ids[a0 + i] - first_expert : 0xFFFFFFFFu;
  const bool valid = e < NE;
  // Entries with no expert here get a key of their own, so that they match nothing.
  const uint32_t same = __match_any_sync(0xffffffffu, valid ? e : NE + lane);
  const uint32_t before = __popc(same & ((1u << lane) - 1));
  __syncthreads();
  if (valid && before == 0) s_cnt[warp * NE + e] = __popc(same);
  __syncthreads();
  if (i < NE) {
    uint32_t run = 0;
    for (uint32_t w = 0; w < 16; w++) {
      const uint32_t c = s_cnt[w * NE + i];
      s_cnt[w * NE + i] = run;
      run += c;
    }
  }
  __syncthreads();
  if (!valid) return;
  uint32_t row = base[e] + chunk_off[(uint64_t)blockIdx.x * NE + e] + s_cnt[warp * NE + e] + before;
  if (group_off) row += group_off[(uint64_t)(blockIdx.x / kScanGroup) * NE + e];
  inv[a0 + i] = row;
  row_src[row] = (a0 + i) / src_div;
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
  dependents_may_launch(), wait_for_predecessors();
  router_topk_block(rl, RouterApprox{}, bias, T, NE, K, ids, w, gs, hist, s_chunk_ids);
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
// One CTA per row. y is f32, or f16 when the tile kernels or other GPUs left it in that form. With res set, the row's
// residual res[t] is added last: a stack's x <- x + block(x) without a kernel of its own.
__device__ __forceinline__ float4 load_row4(const float *y, uint64_t row, uint32_t E, uint32_t i) { return ((const float4 *)(y + row * E))[i]; }
__device__ __forceinline__ float4 load_row4(const __half *y, uint64_t row, uint32_t E, uint32_t i) {
  const uint2 u = ((const uint2 *)(y + row * E))[i];
  const float2 a = __half22float2(*(const __half2 *)&u.x), b = __half22float2(*(const __half2 *)&u.y);
  return make_float4(a.x, a.y, b.x, b.y);
}
template <class Y>
static __global__ void __launch_bounds__(256) k_combine(const Y *__restrict__ y, const uint32_t *__restrict__ inv,
                                                       const float *__restrict__ w, const float *__restrict__ gs,
                                                       const float *__restrict__ s, uint32_t K, uint32_t E, float *__restrict__ out,
                                                       const float *__restrict__ res) {
  dependents_may_launch(), wait_for_predecessors();
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
    if (res) {
      const float4 v = ((const float4 *)(res + (uint64_t)t * E))[i];
      acc.x += v.x, acc.y += v.y, acc.z += v.z, acc.w += v.w;
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
// 256 values. row_stride: bytes from a row to the next when they carry more than the row itself (0: none).
// With place_of, a row goes straight to its places in expert order instead of to its own index: row r has up to
// `places` entries, entry k with an expert when ids[r * places + k] >= 0 and then at row place_of[r * places + k] of
// out's out_rows rows.
static __global__ void __launch_bounds__(256) k_wire_to_f16(const uint8_t *__restrict__ wire, uint32_t K, bool q8k, uint64_t nblk256,
                                                           __half *__restrict__ out, uint32_t row_stride = 0,
                                                           const int32_t *__restrict__ ids = nullptr, const uint32_t *__restrict__ place_of = nullptr,
                                                           uint32_t places = 0, uint64_t out_rows = 0) {
  const uint64_t blk = (uint64_t)blockIdx.x * 8 + threadIdx.x / 32;
  if (blk >= nblk256) return;
  const uint32_t lane = threadIdx.x % 32, per_row = K / 256, wb = row_stride ? row_stride : wire_row_bytes(q8k, K);
  const uint64_t row = blk / per_row;
  const uint32_t b = (uint32_t)(blk % per_row);
  const uint8_t *src = wire + row * wb;
  const char4 lo = ((const char4 *)(src + 256 * b))[2 * lane], hi = ((const char4 *)(src + 256 * b))[2 * lane + 1];
  const float d = q8k ? ((const float *)(src + K))[b] : ((const float *)(src + K))[8 * b + lane / 4];
  const __half2 h0 = __floats2half2_rn(d * (float)lo.x, d * (float)lo.y), h1 = __floats2half2_rn(d * (float)lo.z, d * (float)lo.w);
  const __half2 h2 = __floats2half2_rn(d * (float)hi.x, d * (float)hi.y), h3 = __floats2half2_rn(d * (float)hi.z, d * (float)hi.w);
  uint4 o;
  o.x = *(const uint32_t *)&h0, o.y = *(const uint32_t *)&h1, o.z = *(const uint32_t *)&h2, o.w = *(const uint32_t *)&h3;
  if (!place_of) {
    ((uint4 *)(out + row * K + 256 * b))[lane] = o;
    return;
  }
  // A place past out's rows can only come from an id that is not one of this GPU's experts (the pack leaves such an
  // entry's place unset): it is skipped, not written.
  for (uint32_t k = 0; k < places; k++) {
    if (__ldg(ids + row * places + k) < 0) continue;
    const uint64_t place = __ldg(place_of + row * places + k);
    if (place < out_rows) ((uint4 *)(out + place * K + 256 * b))[lane] = o;
  }
}

// ---------------------------------------------------------------------------------------------------------------
// Expert parallel with one row per (token, GPU). A token's K experts live on a few GPUs (about 5.9 of 8, 2.0 of 2 for
// K = 10 and even routing), so a token's quantised row travels once to each GPU that holds any of its experts, with the
// list of those experts and their routing weights beside it; the GPU returns one row, the weighted sum of its experts'
// results for the token. GPUs own contiguous ranges of `per` experts.
constexpr uint32_t kMaxWorld = 8;
constexpr uint32_t kDestChunk = 256;                   // tokens a CTA plans
constexpr uint32_t kMetaBytes = 2 * 16 + 4 * 16;       // a travelling row's list: 16 u16 local expert ids, 16 f32 weights
__host__ __device__ constexpr uint32_t dispatch_row_bytes(bool q8k, uint32_t K) { return wire_row_bytes(q8k, K) + kMetaBytes; }

// Per chunk of tokens: how many of them go to each GPU, and how many assignments go with them.
static __global__ void __launch_bounds__(kDestChunk) k_dest_count(const int32_t *__restrict__ ids, uint32_t T, uint32_t K, uint32_t per,
                                                                uint32_t *__restrict__ chunk_cnt, uint32_t *__restrict__ chunk_asg) {
  __shared__ uint32_t rows[kMaxWorld], asg[kMaxWorld];
  if (threadIdx.x < kMaxWorld) rows[threadIdx.x] = 0, asg[threadIdx.x] = 0;
  __syncthreads();
  const uint32_t t = blockIdx.x * kDestChunk + threadIdx.x;
  if (t < T) {
    uint32_t mask = 0;
    for (uint32_t k = 0; k < K; k++) {
      const uint32_t g = (uint32_t)ids[(uint64_t)t * K + k] / per;
      atomicAdd(&asg[g], 1u);
      mask |= 1u << g;
    }
    for (uint32_t g = 0; g < kMaxWorld; g++)
      if (mask >> g & 1) atomicAdd(&rows[g], 1u);
  }
  __syncthreads();
  if (threadIdx.x < kMaxWorld) {
    chunk_cnt[blockIdx.x * kMaxWorld + threadIdx.x] = rows[threadIdx.x];
    chunk_asg[blockIdx.x * kMaxWorld + threadIdx.x] = asg[threadIdx.x];
  }
}

// pos[t][g] = the place of token t's row among those this GPU sends to GPU g, in token order, or 0xFFFFFFFF when none
// of its experts lives there. totals[g] = rows for GPU g, totals[kMaxWorld + g] = assignments for it (written by CTA 0).
static __global__ void __launch_bounds__(kDestChunk) k_dest_fill(const int32_t *__restrict__ ids, uint32_t T, uint32_t K, uint32_t per,
                                                               const uint32_t *__restrict__ chunk_cnt, const uint32_t *__restrict__ chunk_asg,
                                                               uint32_t nchunks, uint32_t *__restrict__ pos, uint32_t *__restrict__ totals) {
  __shared__ uint32_t base[kMaxWorld], warp_cnt[kDestChunk / 32][kMaxWorld], tot[2 * kMaxWorld];
  if (threadIdx.x < kMaxWorld) base[threadIdx.x] = 0;
  if (threadIdx.x < 2 * kMaxWorld) tot[threadIdx.x] = 0;
  __syncthreads();
  // The chunks before this one (and, for CTA 0, all of them for the totals).
  for (uint32_t i = threadIdx.x; i < nchunks * kMaxWorld; i += kDestChunk) {
    const uint32_t c = i / kMaxWorld, g = i % kMaxWorld;
    if (c < blockIdx.x && chunk_cnt[i]) atomicAdd(&base[g], chunk_cnt[i]);
    if (blockIdx.x == 0) atomicAdd(&tot[g], chunk_cnt[i]), atomicAdd(&tot[kMaxWorld + g], chunk_asg[i]);
  }
  const uint32_t t = blockIdx.x * kDestChunk + threadIdx.x, lane = threadIdx.x % 32, warp = threadIdx.x / 32;
  uint32_t mask = 0;
  if (t < T)
    for (uint32_t k = 0; k < K; k++) mask |= 1u << ((uint32_t)ids[(uint64_t)t * K + k] / per);
  uint32_t rank[kMaxWorld];
#pragma unroll
  for (uint32_t g = 0; g < kMaxWorld; g++) {
    const uint32_t b = __ballot_sync(0xffffffffu, mask >> g & 1);
    rank[g] = __popc(b & ((1u << lane) - 1));
    if (lane == 0) warp_cnt[warp][g] = __popc(b);
  }
  __syncthreads();
  if (t < T) {
#pragma unroll
    for (uint32_t g = 0; g < kMaxWorld; g++) {
      uint32_t before = base[g];
      for (uint32_t w = 0; w < warp; w++) before += warp_cnt[w][g];
      pos[(uint64_t)t * kMaxWorld + g] = (mask >> g & 1) ? before + rank[g] : 0xFFFFFFFFu;
    }
  }
  if (blockIdx.x == 0 && threadIdx.x < 2 * kMaxWorld) totals[threadIdx.x] = tot[threadIdx.x];
}

// The travelling rows, destination by destination (GPU 0's first), each destination's in token order: the token's
// quantised row as k_gather_wire lays it, then its experts on that GPU as local indices (0xFFFF: none) in rank order,
// then their routing weights. One warp per (token, GPU).
static __global__ void __launch_bounds__(256) k_dispatch_rows(const ActView act, uint32_t E, bool q8k, const int32_t *__restrict__ ids,
                                                             const float *__restrict__ w, const uint32_t *__restrict__ pos,
                                                             const uint32_t *__restrict__ totals, uint32_t T, uint32_t K, uint32_t per,
                                                             uint32_t world, uint8_t *__restrict__ out) {
  const uint32_t lane = threadIdx.x % 32;
  const uint64_t pair = (uint64_t)blockIdx.x * 8 + threadIdx.x / 32;
  if (pair >= (uint64_t)T * world) return;
  const uint32_t t = (uint32_t)(pair / world), g = (uint32_t)(pair % world), p = pos[(uint64_t)t * kMaxWorld + g];
  if (p == 0xFFFFFFFFu) return;
  uint32_t first = 0;
  for (uint32_t i = 0; i < g; i++) first += totals[i];
  const uint32_t wb = wire_row_bytes(q8k, E), dbytes = q8k ? E / 64 : E / 8;
  uint8_t *dst = out + (uint64_t)(first + p) * (wb + kMetaBytes);
  const int4 *q = (const int4 *)(act.q + (uint64_t)t * act.q_stride);
  for (uint32_t i = lane; i < E / 16; i += 32) ((int4 *)dst)[i] = q[i];
  const uint32_t *d = (const uint32_t *)((const uint8_t *)act.d + (uint64_t)t * act.d_stride);
  for (uint32_t i = lane; i < dbytes / 4; i += 32) ((uint32_t *)(dst + E))[i] = d[i];
  if (q8k) {
    const uint32_t *b = (const uint32_t *)((const uint8_t *)act.bs + (uint64_t)t * act.bs_stride);
    for (uint32_t i = lane; i < E / 32; i += 32) ((uint32_t *)(dst + E + dbytes))[i] = b[i];
  }
  if (lane < 16) {
    uint32_t local = 0xFFFFu;
    float wk = 0.0f;
    if (lane < K) {
      const uint32_t e = (uint32_t)ids[(uint64_t)t * K + lane];
      if (e / per == g) local = e % per, wk = w[(uint64_t)t * K + lane];
    }
    ((uint16_t *)(dst + wb))[lane] = (uint16_t)local;
    ((float *)(dst + wb + 32))[lane] = wk;
  }
}

// The lists of the rows received, flattened: ids[r * K + k] = first_expert + the local index, or -1 for no expert;
// w[r * K + k] its weight. One thread per entry.
static __global__ void __launch_bounds__(256) k_meta_unpack(const uint8_t *__restrict__ rows, uint64_t R, uint32_t wb, uint32_t K,
                                                           uint32_t first_expert, int32_t *__restrict__ ids, float *__restrict__ w) {
  const uint64_t i = (uint64_t)blockIdx.x * 256 + threadIdx.x;
  if (i >= R * K) return;
  const uint8_t *meta = rows + (i / K) * (wb + kMetaBytes) + wb;
  const uint32_t local = ((const uint16_t *)meta)[i % K];
  ids[i] = local == 0xFFFFu ? -1 : (int32_t)(first_expert + local);
  w[i] = ((const float *)(meta + 32))[i % K];
}

// What a GPU returns for a received row: the weighted sum of its experts' results for the row, in the row's rank
// order, f32 accumulate, as f16. One CTA per row.
template <class Y>
static __global__ void __launch_bounds__(256) k_combine_partial(const Y *__restrict__ y, const uint32_t *__restrict__ inv,
                                                               const int32_t *__restrict__ ids, const float *__restrict__ w, uint32_t K,
                                                               uint32_t E, __half *__restrict__ out) {
  const uint64_t r = blockIdx.x;
  __shared__ uint32_t rows[16];
  __shared__ float wk[16];
  __shared__ uint32_t n;
  if (threadIdx.x == 0) {
    uint32_t m = 0;
    for (uint32_t k = 0; k < K; k++)
      if (ids[r * K + k] >= 0) rows[m] = inv[r * K + k], wk[m] = w[r * K + k], m++;
    n = m;
  }
  __syncthreads();
  for (uint32_t i = threadIdx.x; i < E / 4; i += 256) {
    float4 acc = make_float4(0, 0, 0, 0);
    for (uint32_t k = 0; k < n; k++) {
      const float4 v = load_row4(y, rows[k], E, i);
      acc.x = fmaf(wk[k], v.x, acc.x), acc.y = fmaf(wk[k], v.y, acc.y);
      acc.z = fmaf(wk[k], v.z, acc.z), acc.w = fmaf(wk[k], v.w, acc.w);
    }
    const __half2 a = __floats2half2_rn(acc.x, acc.y), b = __floats2half2_rn(acc.z, acc.w);
    uint2 o;
    o.x = *(const uint32_t *)&a, o.y = *(const uint32_t *)&b;
    ((uint2 *)(out + r * E))[i] = o;
  }
}

// At home: out[t] = the GPUs' partial sums for token t added in GPU order, + gs[t] * s[t] (+ res[t]). back holds the
// rows as they were sent: destination by destination. One CTA per token.
static __global__ void __launch_bounds__(256) k_combine_home(const __half *__restrict__ back, const uint32_t *__restrict__ pos,
                                                            const uint32_t *__restrict__ totals, const float *__restrict__ gs,
                                                            const float *__restrict__ s, const float *__restrict__ res, uint32_t world,
                                                            uint32_t E, float *__restrict__ out) {
  const uint32_t t = blockIdx.x;
  __shared__ uint32_t rows[kMaxWorld];
  __shared__ uint32_t n;
  if (threadIdx.x == 0) {
    uint32_t m = 0, first = 0;
    for (uint32_t g = 0; g < world; g++) {
      const uint32_t p = pos[(uint64_t)t * kMaxWorld + g];
      if (p != 0xFFFFFFFFu) rows[m++] = first + p;
      first += totals[g];
    }
    n = m;
  }
  __syncthreads();
  const float g = s ? gs[t] : 0.0f;
  for (uint32_t i = threadIdx.x; i < E / 4; i += 256) {
    float4 acc = make_float4(0, 0, 0, 0);
    for (uint32_t k = 0; k < n; k++) {
      const float4 v = load_row4(back, rows[k], E, i);
      acc.x += v.x, acc.y += v.y, acc.z += v.z, acc.w += v.w;
    }
    if (s) {
      const float4 v = ((const float4 *)(s + (uint64_t)t * E))[i];
      acc.x = fmaf(g, v.x, acc.x), acc.y = fmaf(g, v.y, acc.y), acc.z = fmaf(g, v.z, acc.z), acc.w = fmaf(g, v.w, acc.w);
    }
    if (res) {
      const float4 v = ((const float4 *)(res + (uint64_t)t * E))[i];
      acc.x += v.x, acc.y += v.y, acc.z += v.z, acc.w += v.w;
    }
    ((float4 *)(out + (uint64_t)t * E))[i] = acc;
  }
}

// out[r] = y[inv[r]]: the experts' rows back in the order they arrived, f32 or f16 on either side. One CTA per row.
template <class Y, class O>
static __global__ void __launch_bounds__(256) k_unpermute(const Y *__restrict__ y, const uint32_t *__restrict__ inv, uint32_t E,
                                                         O *__restrict__ out) {
  const uint64_t r = blockIdx.x, src = inv[r];
  for (uint32_t i = threadIdx.x; i < E / 4; i += 256) {
    if constexpr (sizeof(Y) == 2 && sizeof(O) == 2) {
      ((uint2 *)(out + r * E))[i] = ((const uint2 *)(y + src * E))[i];
    } else {
      const float4 v = load_row4(y, src, E, i);
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
}

}  // namespace moe
