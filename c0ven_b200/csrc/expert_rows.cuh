// The experts' products for few rows per expert: integer dots of quantised weights against int8 activations, a group
// of lanes per weight row, 128-bit loads of the quants in the runs layout, the weights decoded once in registers for
// every row of the group, shuffle reductions. This is the bandwidth-bound path (decode and draft-verify steps); it
// replaces the reference's grouped GEMVs (kernels/quant/moe.cl:230-302,416-471; kernels/quant/matvec.cl:101-159) and
// follows the arithmetic of its CPU path (core/cpu/experts.cpp:152-284): activations as q8_0 or q8_K, integer block
// sums, f32 scales.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdint>

#include "cuda_rt.h"
#include "formats.h"
#include "iq4nl_values.h"

namespace moe {

// Rows start .. start + n of the expert order, all of one expert (its slot among this GPU's experts), n <= 8: the
// reference's MoeGroup (shared/moe_tile.h:20-33) with the rows named by their place in expert order.
struct MoeGroup {
  uint32_t slot, start, n;
};
constexpr int kGroupMax = 8;

// Quantised activation rows: a row's K codes at q + row * q_stride; its scales at d + row * d_stride bytes (q8_0: K/32
// floats, the f16 scale widened; q8_K: K/256 floats); q8_K's sums of each 16 codes at bs + row * bs_stride bytes. The
// strides let the three parts be arrays of their own or pieces of one packed row.
struct ActView {
  const int8_t *q;
  const float *d;
  const int16_t *bs;
  uint32_t q_stride, d_stride, bs_stride;
};

struct ExpertRowsArgs {
  const uint8_t *w0, *w1;  // slot 0's slice of the matrix (gate, up) or (down, unused), runs layout
  uint64_t slice_bytes;    // from one slot's slice to the next
  uint32_t K, R;           // values per weight row; weight rows
  uint32_t rows_per_cta;
  ActView act;
  const uint32_t *act_row;  // expert-order row -> activation row; null: the same row
  const MoeGroup *groups;   // null: dense_rows rows of slot 0, taken M at a time
  const uint32_t *ngroups;
  uint32_t dense_rows;
  uint32_t slabs;           // row slabs a CTA takes one after another (0 or 1: one); only with the row length known at compile time
  float *out;  // out[expert-order row][r]
  uint32_t out_stride;
  float limit;  // SwiGLU limit, 0: off
};

__device__ __forceinline__ uint4 ldg_stream16(const void *p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
__device__ __forceinline__ int dot4x4(const uint4 &w, const int4 &a) {
  int s = __dp4a((int)w.x, a.x, 0);
  s = __dp4a((int)w.y, a.y, s);
  s = __dp4a((int)w.z, a.z, s);
  return __dp4a((int)w.w, a.w, s);
}

// Bytes of one activation row in shared memory: codes, then the scales (padded to 16), then q8_K's sums.
__host__ __device__ constexpr uint32_t act_d_bytes(bool q8k, uint32_t K) { return q8k ? ((K / 64 + 15) & ~15u) : K / 8; }
constexpr uint32_t kRowsMaxK = 16384;  // the longest activation row the integer-dot kernels stage (8 rows of it fit an SM's shared memory)
__host__ __device__ constexpr uint32_t act_row_stride(bool q8k, uint32_t K) { return K + act_d_bytes(q8k, K) + (q8k ? K / 8 : 0) + 16; }

// SwiGLU as the CPU path states it (core/cpu/experts.cpp:21-27).
__device__ __forceinline__ float swiglu(float g, float u, float limit) {
  if (limit > 0.0f) {
    g = fminf(g, limit);
    u = fminf(fmaxf(u, -limit), limit);
  }
  return g / (1.0f + expf(-g)) * u;
}

// One lane's unit of a weight row: what it loads (Raw, 16 bytes of quants and the scales beside them) and its dot with
// the matching codes of M activation rows. nblk: blocks in the slice; r: row; u: unit within the row.
template <int QT>
struct Unit;

// Q8_0: y = d * q (docs/spec/QUANT_FORMATS.md:461). A unit is 16 codes, half a block.
template <>
struct Unit<QT_Q8_0> {
  static constexpr int kValues = 16;
  struct Raw {
    uint4 q;
    float d;
  };
  __device__ static __forceinline__ Raw fetch(const uint8_t *s, uint64_t nblk, uint32_t K, uint32_t r, uint32_t u, const uint32_t *) {
    Raw x;
    x.q = ldg_stream16(s + (uint64_t)r * K + 16u * u);
    x.d = __half2float(__ldg((const __half *)(s + 32 * nblk) + (uint64_t)r * (K / 32) + u / 2));
    return x;
  }
  template <int M>
  __device__ static __forceinline__ void dot(const Raw &x, uint32_t K, uint32_t u, const uint8_t *acts, uint32_t stride, float *acc, uint32_t n) {
#pragma unroll
    for (int t = 0; t < M; t++) {
      if ((uint32_t)t >= n) break;  // the group's rows: the same for the whole CTA
      const uint8_t *a = acts + t * stride;
      const int s = dot4x4(x.q, *(const int4 *)(a + 16u * u));
      acc[t] = fmaf(x.d * ((const float *)(a + K))[u / 2], (float)s, acc[t]);
    }
  }
};

// Q4_K: y = d * sc * q - dmin * m, eight sub-blocks of 32 with 6-bit sc and m (QUANT_FORMATS.md:373-394). A unit is
// 16 bytes of qs: 16 values of sub-block 2p in the low nibbles, 16 of sub-block 2p + 1 in the high ones.
template <>
struct Unit<QT_Q4_K> {
  static constexpr int kValues = 32;
  struct Raw {
    uint4 q;
    uint32_t s0, s1, s2;
    __half2 dm;
  };
  __device__ static __forceinline__ Raw fetch(const uint8_t *s, uint64_t nblk, uint32_t K, uint32_t r, uint32_t u, const uint32_t *) {
    Raw x;
    x.q = ldg_stream16(s + (uint64_t)r * (K / 2) + 16u * u);
    const uint64_t blk = (uint64_t)r * (K / 256) + u / 8;
    const uint4 hd = __ldg((const uint4 *)(s + 128 * nblk + 16 * blk));  // d, dmin, then the 12 bytes of scales
    x.dm = *(const __half2 *)&hd.x;
    x.s0 = hd.y, x.s1 = hd.z, x.s2 = hd.w;
    return x;
  }
  __device__ static __forceinline__ uint32_t byte_of(const Raw &x, int i) {
    const uint32_t w = i < 4 ? x.s0 : i < 8 ? x.s1 : x.s2;
    return (w >> (8 * (i & 3))) & 0xFF;
  }
  // The packed scale and minimum of sub-block j (QUANT_FORMATS.md:386-392).
  __device__ static __forceinline__ void scale_min(const Raw &x, int j, int &sc, int &m) {
    if (j < 4) {
      sc = byte_of(x, j) & 63;
      m = byte_of(x, j + 4) & 63;
    } else {
      sc = (byte_of(x, j + 4) & 0xF) | ((byte_of(x, j - 4) >> 6) << 4);
      m = (byte_of(x, j + 4) >> 4) | ((byte_of(x, j) >> 6) << 4);
    }
  }
  template <int M>
  __device__ static __forceinline__ void dot(const Raw &x, uint32_t K, uint32_t u, const uint8_t *acts, uint32_t stride, float *acc, uint32_t n) {
    const uint32_t b = u / 8, j = u % 8, p = j / 2, hf = j & 1;
    int sc_lo, m_lo, sc_hi, m_hi;
    scale_min(x, 2 * p, sc_lo, m_lo);
    scale_min(x, 2 * p + 1, sc_hi, m_hi);
    const uint4 lo = make_uint4(x.q.x & 0x0F0F0F0Fu, x.q.y & 0x0F0F0F0Fu, x.q.z & 0x0F0F0F0Fu, x.q.w & 0x0F0F0F0Fu);
    const uint4 hi = make_uint4((x.q.x >> 4) & 0x0F0F0F0Fu, (x.q.y >> 4) & 0x0F0F0F0Fu, (x.q.z >> 4) & 0x0F0F0F0Fu,
                                (x.q.w >> 4) & 0x0F0F0F0Fu);
    const float d = __low2float(x.dm), dmin = __high2float(x.dm);
    const uint32_t dsz = act_d_bytes(true, K);
#pragma unroll
    for (int t = 0; t < M; t++) {
      if ((uint32_t)t >= n) break;  // the group's rows: the same for the whole CTA
      const uint8_t *a = acts + t * stride;
      const uint8_t *av = a + 256 * b + 64 * p + 16 * hf;
      const int s_lo = dot4x4(lo, *(const int4 *)av), s_hi = dot4x4(hi, *(const int4 *)(av + 32));
      const int16_t *bs = (const int16_t *)(a + K + dsz) + 16 * b + 4 * p + hf;
      const float da = ((const float *)(a + K))[b];
      acc[t] += da * (d * (float)(sc_lo * s_lo + sc_hi * s_hi) - dmin * (float)(m_lo * bs[0] + m_hi * bs[2]));
    }
  }
};

// Q6_K: y = d * scales[v / 16] * (q - 32), 6-bit codes split into ql (low 4) and qh (high 2) (QUANT_FORMATS.md:419-441).
// A unit is 16 bytes of ql with the 16 bytes of qh that complete them: 16 values in the low nibbles and 16 in the high
// ones, each a whole group of 16 with its own int8 scale.
template <>
struct Unit<QT_Q6_K> {
  static constexpr int kValues = 32;
  struct Raw {
    uint4 ql, qh;
    int sc_lo, sc_hi;
    float d;
  };
  __device__ static __forceinline__ Raw fetch(const uint8_t *s, uint64_t nblk, uint32_t K, uint32_t r, uint32_t u, const uint32_t *) {
    Raw x;
    x.ql = ldg_stream16(s + (uint64_t)r * (K / 2) + 16u * u);
    const uint32_t j = u % 8, h = j / 4, jj = j % 4;
    const uint64_t blk = (uint64_t)r * (K / 256) + u / 8;
    x.qh = ldg_stream16(s + 128 * nblk + 64 * blk + 32 * h + 16 * (jj & 1));
    const int8_t *sc = (const int8_t *)(s + 192 * nblk + 16 * blk) + 8 * h + 2 * (jj >> 1) + (jj & 1);
    x.sc_lo = __ldg(sc), x.sc_hi = __ldg(sc + 4);
    x.d = __half2float(__ldg((const __half *)(s + 208 * nblk) + blk));
    return x;
  }
  template <int M>
  __device__ static __forceinline__ void dot(const Raw &x, uint32_t K, uint32_t u, const uint8_t *acts, uint32_t stride, float *acc, uint32_t n) {
    const uint32_t b = u / 8, j = u % 8, h = j / 4, jj = j % 4, sh = jj < 2 ? 0 : 2;
    const uint32_t g16 = 8 * h + 2 * (jj >> 1) + (jj & 1);  // the low nibbles' group of 16; the high ones' is 4 on
    uint4 lo, hi;
    lo.x = (x.ql.x & 0x0F0F0F0Fu) | (((x.qh.x >> sh) & 0x03030303u) << 4);
    lo.y = (x.ql.y & 0x0F0F0F0Fu) | (((x.qh.y >> sh) & 0x03030303u) << 4);
    lo.z = (x.ql.z & 0x0F0F0F0Fu) | (((x.qh.z >> sh) & 0x03030303u) << 4);
    lo.w = (x.ql.w & 0x0F0F0F0Fu) | (((x.qh.w >> sh) & 0x03030303u) << 4);
    hi.x = ((x.ql.x >> 4) & 0x0F0F0F0Fu) | (((x.qh.x >> (sh + 4)) & 0x03030303u) << 4);
    hi.y = ((x.ql.y >> 4) & 0x0F0F0F0Fu) | (((x.qh.y >> (sh + 4)) & 0x03030303u) << 4);
    hi.z = ((x.ql.z >> 4) & 0x0F0F0F0Fu) | (((x.qh.z >> (sh + 4)) & 0x03030303u) << 4);
    hi.w = ((x.ql.w >> 4) & 0x0F0F0F0Fu) | (((x.qh.w >> (sh + 4)) & 0x03030303u) << 4);
    const uint32_t dsz = act_d_bytes(true, K);
#pragma unroll
    for (int t = 0; t < M; t++) {
      if ((uint32_t)t >= n) break;  // the group's rows: the same for the whole CTA
      const uint8_t *a = acts + t * stride;
      const uint8_t *av = a + 256 * b + 16 * g16;
      const int s_lo = dot4x4(lo, *(const int4 *)av), s_hi = dot4x4(hi, *(const int4 *)(av + 64));
      const int16_t *bs = (const int16_t *)(a + K + dsz) + 16 * b + g16;
      const int isum = x.sc_lo * (s_lo - 32 * bs[0]) + x.sc_hi * (s_hi - 32 * bs[4]);
      acc[t] = fmaf(x.d * ((const float *)(a + K))[b], (float)isum, acc[t]);
    }
  }
};

// IQ3_S: y = d * (1 + 2 s) * grid[index][i] * sign, 9-bit indices into the 512-entry codebook, one per 4 values
// (QUANT_FORMATS.md:178-207). A unit is 16 bytes of qs: two sub-blocks of 32. The codebook sits in shared memory; the
// signs go onto the codebook's bytes once, for every activation row.
template <>
struct Unit<QT_IQ3_S> {
  static constexpr int kValues = 64;
  struct Raw {
    uint4 qs;
    uint2 sg;
    uint32_t qh, sc;
    float d;
  };
  __device__ static __forceinline__ Raw fetch(const uint8_t *s, uint64_t nblk, uint32_t K, uint32_t r, uint32_t u, const uint32_t *) {
    Raw x;
    x.qs = ldg_stream16(s + (uint64_t)r * (K / 4) + 16u * u);
    const uint32_t c = u % 4;
    const uint64_t blk = (uint64_t)r * (K / 256) + u / 4;
    x.sg = __ldg((const uint2 *)(s + 64 * nblk + 32 * blk + 8 * c));
    x.qh = __ldg((const uint16_t *)(s + 96 * nblk + 8 * blk + 2 * c));
    x.sc = __ldg(s + 104 * nblk + 4 * blk + c);
    x.d = __half2float(__ldg((const __half *)(s + 108 * nblk) + blk));
    return x;
  }
  template <int M>
  __device__ static __forceinline__ void dot(const Raw &x, uint32_t K, uint32_t u, const uint8_t *acts, uint32_t stride, float *acc,
                                             uint32_t n, const uint32_t *grid) {
    const uint32_t b = u / 4, c = u % 4;
    // A codebook word is four values in 1 .. 15; a sign bit negates its byte: (v ^ 0xFF) + 1 = 256 - v stays within the
    // byte for v >= 1, so the four bytes take one exclusive-or and one 32-bit add. The nibble's bits reach the bytes'
    // low bits by one multiply: bit i times 2^(7 i) lands on bit 8 i, and no two products share a bit.
    int g[16];
    const uint32_t qh9 = x.qh << 8;
#pragma unroll
    for (int i = 0; i < 16; i++) {
      const uint32_t word = i < 4 ? x.qs.x : i < 8 ? x.qs.y : i < 12 ? x.qs.z : x.qs.w;
      const uint32_t idx = ((word >> (8 * (i & 3))) & 0xFF) | ((qh9 >> i) & 0x100u);
      const uint32_t nib = ((i < 8 ? x.sg.x : x.sg.y) >> (4 * (i & 7))) & 0xF;
      const uint32_t lsb = (nib * 0x00204081u) & 0x01010101u;
      g[i] = (int)((grid[idx] ^ (lsb * 0xFFu)) + lsb);
    }
    const int sc0 = 2 * (int)(x.sc & 0xF) + 1, sc1 = 2 * (int)((x.sc >> 4) & 0xF) + 1;
#pragma unroll
    for (int t = 0; t < M; t++) {
      if ((uint32_t)t >= n) break;  // the group's rows: the same for the whole CTA
      const uint8_t *a = acts + t * stride;
      const int4 *av = (const int4 *)(a + 256 * b + 64 * c);
      const uint32_t sw = (u >> 1) & 3;  // act_slot's swizzle
      const int4 a0 = av[0 ^ sw], a1 = av[1 ^ sw], a2 = av[2 ^ sw], a3 = av[3 ^ sw];
      int s0 = __dp4a(g[0], a0.x, 0), s1 = __dp4a(g[8], a2.x, 0);
      s0 = __dp4a(g[1], a0.y, s0), s1 = __dp4a(g[9], a2.y, s1);
      s0 = __dp4a(g[2], a0.z, s0), s1 = __dp4a(g[10], a2.z, s1);
      s0 = __dp4a(g[3], a0.w, s0), s1 = __dp4a(g[11], a2.w, s1);
      s0 = __dp4a(g[4], a1.x, s0), s1 = __dp4a(g[12], a3.x, s1);
      s0 = __dp4a(g[5], a1.y, s0), s1 = __dp4a(g[13], a3.y, s1);
      s0 = __dp4a(g[6], a1.z, s0), s1 = __dp4a(g[14], a3.z, s1);
      s0 = __dp4a(g[7], a1.w, s0), s1 = __dp4a(g[15], a3.w, s1);
      acc[t] = fmaf(x.d * ((const float *)(a + K))[b], (float)(sc0 * s0 + sc1 * s1), acc[t]);
    }
  }
};

// A codebook word's four bytes made negative where the nibble's bits say so. A byte is in 1 .. 127, so (v ^ 0xFF) + 1 =
// 256 - v stays within the byte and the four take one exclusive-or and one 32-bit add; the nibble's bits reach the
// bytes' low bits by one multiply: bit i times 2^(7 i) lands on bit 8 i, and no two products share a bit.
__device__ __forceinline__ int signed_word(uint32_t g, uint32_t nib) {
  const uint32_t lsb = (nib * 0x00204081u) & 0x01010101u;
  return (int)((g ^ (lsb * 0xFFu)) + lsb);
}
// 8 activation words of a sub-block against 8 decoded words.
__device__ __forceinline__ int dot8(const int *g, const int4 &a0, const int4 &a1) {
  int s = __dp4a(g[0], a0.x, 0);
  s = __dp4a(g[1], a0.y, s), s = __dp4a(g[2], a0.z, s), s = __dp4a(g[3], a0.w, s);
  s = __dp4a(g[4], a1.x, s), s = __dp4a(g[5], a1.y, s), s = __dp4a(g[6], a1.z, s), s = __dp4a(g[7], a1.w, s);
  return s;
}

// IQ3_XXS: y = d * (0.5 + s) / 2 * grid[index][i] * sign: 8-bit indices into a 256-entry codebook, one per 4 values;
// a sub-block of 32 has one word: four 7-bit sign indices (the eighth sign of each 8 values is the index's parity)
// and the 4-bit s (QUANT_FORMATS.md:147-173). A unit is 16 bytes of indices: two sub-blocks.
template <>
struct Unit<QT_IQ3_XXS> {
  static constexpr int kValues = 64;
  struct Raw {
    uint4 qs;
    uint2 gas;
    float d;
  };
  __device__ static __forceinline__ Raw fetch(const uint8_t *s, uint64_t nblk, uint32_t K, uint32_t r, uint32_t u, const uint32_t *) {
    Raw x;
    x.qs = ldg_stream16(s + (uint64_t)r * (K / 4) + 16u * u);
    const uint32_t c = u % 4;
    const uint64_t blk = (uint64_t)r * (K / 256) + u / 4;
    x.gas = __ldg((const uint2 *)(s + 64 * nblk + 32 * blk + 8 * c));
    x.d = 0.25f * __half2float(__ldg((const __half *)(s + 96 * nblk) + blk));  // (2 s + 1) / 4 = (0.5 + s) / 2
    return x;
  }
  template <int M>
  __device__ static __forceinline__ void dot(const Raw &x, uint32_t K, uint32_t u, const uint8_t *acts, uint32_t stride, float *acc,
                                             uint32_t n, const uint32_t *grid) {
    const uint32_t b = u / 4, c = u % 4;
    int g[16];
#pragma unroll
    for (int i = 0; i < 16; i++) {
      const uint32_t word = i < 4 ? x.qs.x : i < 8 ? x.qs.y : i < 12 ? x.qs.z : x.qs.w;
      const uint32_t w32 = i < 8 ? x.gas.x : x.gas.y;
      const uint32_t k7 = (w32 >> (7 * ((i & 7) >> 1))) & 127u, sbyte = k7 | ((__popc(k7) & 1u) << 7);
      g[i] = signed_word(grid[(word >> (8 * (i & 3))) & 0xFF], (sbyte >> (4 * (i & 1))) & 0xF);
    }
    const int sc0 = 2 * (int)(x.gas.x >> 28) + 1, sc1 = 2 * (int)(x.gas.y >> 28) + 1;
#pragma unroll
    for (int t = 0; t < M; t++) {
      if ((uint32_t)t >= n) break;  // the group's rows: the same for the whole CTA
      const uint8_t *a = acts + t * stride;
      const int4 *av = (const int4 *)(a + 256 * b + 64 * c);
      const uint32_t sw = (u >> 1) & 3;  // act_slot's swizzle
      const int s0 = dot8(g, av[0 ^ sw], av[1 ^ sw]), s1 = dot8(g + 8, av[2 ^ sw], av[3 ^ sw]);
      acc[t] = fmaf(x.d * ((const float *)(a + K))[b], (float)(sc0 * s0 + sc1 * s1), acc[t]);
    }
  }
};

// IQ2_S: y = d * (0.5 + s) / 4 * grid[index][i] * sign: 10-bit indices into a 1024-entry codebook of 8 values (8 bits in
// qs, 2 in qh), a byte of signs a group, a 4-bit s per 16 values (QUANT_FORMATS.md:115-145). A unit is 8 bytes of qs:
// two sub-blocks of 32. The codebook in shared memory is two words an entry.
template <>
struct Unit<QT_IQ2_S> {
  static constexpr int kValues = 64;
  struct Raw {
    uint2 qs, sg;
    uint32_t qh, sc;
    float d;
  };
  __device__ static __forceinline__ Raw fetch(const uint8_t *s, uint64_t nblk, uint32_t K, uint32_t r, uint32_t u, const uint32_t *) {
    Raw x;
    x.qs = __ldg((const uint2 *)(s + (uint64_t)r * (K / 8) + 8u * u));
    const uint32_t c = u % 4;
    const uint64_t blk = (uint64_t)r * (K / 256) + u / 4;
    x.sg = __ldg((const uint2 *)(s + 32 * nblk + 32 * blk + 8 * c));
    x.qh = __ldg((const uint16_t *)(s + 64 * nblk + 8 * blk + 2 * c));
    x.sc = __ldg((const uint16_t *)(s + 72 * nblk + 8 * blk + 2 * c));
    x.d = 0.125f * __half2float(__ldg((const __half *)(s + 80 * nblk) + blk));  // (2 s + 1) / 8 = (0.5 + s) / 4
    return x;
  }
  template <int M>
  __device__ static __forceinline__ void dot(const Raw &x, uint32_t K, uint32_t u, const uint8_t *acts, uint32_t stride, float *acc,
                                             uint32_t n, const uint32_t *grid) {
    const uint32_t b = u / 4, c = u % 4;
    const uint2 *grid2 = (const uint2 *)grid;
    int g[16];
#pragma unroll
    for (int j = 0; j < 8; j++) {  // group j: sub-block j / 4, its group j % 4
      const uint32_t lo8 = ((j < 4 ? x.qs.x : x.qs.y) >> (8 * (j & 3))) & 0xFF;
      const uint32_t hi2 = ((x.qh >> (8 * (j >> 2))) >> (2 * (j & 3))) & 3u;
      const uint32_t sb = ((j < 4 ? x.sg.x : x.sg.y) >> (8 * (j & 3))) & 0xFF;
      const uint2 e = grid2[lo8 | (hi2 << 8)];
      g[2 * j] = signed_word(e.x, sb & 0xF), g[2 * j + 1] = signed_word(e.y, sb >> 4);
    }
    // 2 s + 1 of the four 16-value halves.
    const int k0 = 2 * (int)(x.sc & 0xF) + 1, k1 = 2 * (int)((x.sc >> 4) & 0xF) + 1, k2 = 2 * (int)((x.sc >> 8) & 0xF) + 1,
              k3 = 2 * (int)((x.sc >> 12) & 0xF) + 1;
#pragma unroll
    for (int t = 0; t < M; t++) {
      if ((uint32_t)t >= n) break;  // the group's rows: the same for the whole CTA
      const uint8_t *a = acts + t * stride;
      const int4 *av = (const int4 *)(a + 256 * b + 64 * c);
      const uint32_t sw = (u >> 1) & 3;  // act_slot's swizzle
      const int4 a0 = av[0 ^ sw], a1 = av[1 ^ sw], a2 = av[2 ^ sw], a3 = av[3 ^ sw];
      int p0 = __dp4a(g[0], a0.x, 0), p1 = __dp4a(g[4], a1.x, 0), p2 = __dp4a(g[8], a2.x, 0), p3 = __dp4a(g[12], a3.x, 0);
      p0 = __dp4a(g[1], a0.y, p0), p1 = __dp4a(g[5], a1.y, p1), p2 = __dp4a(g[9], a2.y, p2), p3 = __dp4a(g[13], a3.y, p3);
      p0 = __dp4a(g[2], a0.z, p0), p1 = __dp4a(g[6], a1.z, p1), p2 = __dp4a(g[10], a2.z, p2), p3 = __dp4a(g[14], a3.z, p3);
      p0 = __dp4a(g[3], a0.w, p0), p1 = __dp4a(g[7], a1.w, p1), p2 = __dp4a(g[11], a2.w, p2), p3 = __dp4a(g[15], a3.w, p3);
      acc[t] = fmaf(x.d * ((const float *)(a + K))[b], (float)(k0 * p0 + k1 * p1 + k2 * p2 + k3 * p3), acc[t]);
    }
  }
};

// The 16-entry table of IQ4_NL and IQ4_XS as four words of four signed bytes, entries 4 i .. 4 i + 3 in word i.
__host__ __device__ constexpr uint32_t iq4_table_word(int i) {
  return (uint32_t)(uint8_t)kIq4nlValues[4 * i] | (uint32_t)(uint8_t)kIq4nlValues[4 * i + 1] << 8 | (uint32_t)(uint8_t)kIq4nlValues[4 * i + 2] << 16 |
         (uint32_t)(uint8_t)kIq4nlValues[4 * i + 3] << 24;
}
// Table values of the eight nibbles of q: lo = those of its four bytes' low nibbles (byte order kept), hi = of the
// high ones. A byte permute looks four nibbles up at once: its selector's digits are the nibbles' low three bits
// (entries 0 .. 7 from the table's first two words, 8 .. 15 from its last two), and a second permute takes each
// byte from the one or the other by the nibble's fourth bit. A third pair of permutes parts even nibbles from odd.
__device__ __forceinline__ void iq4_lookup8(uint32_t q, uint32_t &lo, uint32_t &hi) {
  constexpr uint32_t T0 = iq4_table_word(0), T1 = iq4_table_word(1), T2 = iq4_table_word(2), T3 = iq4_table_word(3);
  const uint32_t qa = q & 0xFFFFu, qb = q >> 16;
  const uint32_t sa = qa & 0x7777u, sb = qb & 0x7777u;
  const uint32_t r0 = __byte_perm(__byte_perm(T0, T1, sa), __byte_perm(T2, T3, sa), 0x3210u | ((qa & 0x8888u) >> 1));
  const uint32_t r1 = __byte_perm(__byte_perm(T0, T1, sb), __byte_perm(T2, T3, sb), 0x3210u | ((qb & 0x8888u) >> 1));
  lo = __byte_perm(r0, r1, 0x6420u), hi = __byte_perm(r0, r1, 0x7531u);
}

// Sixteen 2-bit codes (a word's low or high half: 4 bytes of 4 codes) as 16 signed bytes q - 1 in four words. A byte's
// four codes are spread to the digits of a permute selector, whose table is the bytes -1, 0, 1, 2.
__device__ __forceinline__ uint32_t q2_bytes(uint32_t c) {  // c: one byte, four codes
  const uint32_t sel = (c & 0x3u) | ((c & 0xCu) << 2) | ((c & 0x30u) << 4) | ((c & 0xC0u) << 6);
  return __byte_perm(0x020100FFu, 0u, sel);
}

// Q2_0: y = (q - 1) * d, 64 values in 16 bytes with an f16 scale, value j in bits 2 (j mod 4) of byte j / 4
// (QUANT_FORMATS.md:251-270). A unit is one block; it meets two q8_0 blocks of activations, each with its own scale.
template <>
struct Unit<QT_Q2_0> {
  static constexpr int kValues = 64;
  struct Raw {
    uint4 q;
    float d;
  };
  __device__ static __forceinline__ Raw fetch(const uint8_t *s, uint64_t nblk, uint32_t K, uint32_t r, uint32_t u, const uint32_t *) {
    Raw x;
    x.q = ldg_stream16(s + (uint64_t)r * (K / 4) + 16u * u);
    x.d = __half2float(__ldg((const __half *)(s + 16 * nblk) + (uint64_t)r * (K / 64) + u));
    return x;
  }
  template <int M>
  __device__ static __forceinline__ void dot(const Raw &x, uint32_t K, uint32_t u, const uint8_t *acts, uint32_t stride, float *acc, uint32_t n) {
    int g[16];
#pragma unroll
    for (int i = 0; i < 16; i++) {
      const uint32_t word = i < 4 ? x.q.x : i < 8 ? x.q.y : i < 12 ? x.q.z : x.q.w;
      g[i] = (int)q2_bytes((word >> (8 * (i & 3))) & 0xFF);
    }
#pragma unroll
    for (int t = 0; t < M; t++) {
      if ((uint32_t)t >= n) break;  // the group's rows: the same for the whole CTA
      const uint8_t *a = acts + t * stride;
      const int4 *av = (const int4 *)(a + 64u * u);
      const int s0 = dot8(g, av[0], av[1]), s1 = dot8(g + 8, av[2], av[3]);
      const float *da = (const float *)(a + K) + 2 * u;
      acc[t] = fmaf(x.d * da[0], (float)s0, acc[t]);
      acc[t] = fmaf(x.d * da[1], (float)s1, acc[t]);
    }
  }
};

// IQ4_NL: y = d * table[q], blocks of 32 with an f16 scale; a block's 16 bytes hold values 0 .. 15 in their low nibbles
// and 16 .. 31 in their high ones (QUANT_FORMATS.md:236-247). A unit is one block. Activations are q8_0.
template <>
struct Unit<QT_IQ4_NL> {
  static constexpr int kValues = 32;
  struct Raw {
    uint4 q;
    float d;
  };
  __device__ static __forceinline__ Raw fetch(const uint8_t *s, uint64_t nblk, uint32_t K, uint32_t r, uint32_t u, const uint32_t *) {
    Raw x;
    x.q = ldg_stream16(s + (uint64_t)r * (K / 2) + 16u * u);
    x.d = __half2float(__ldg((const __half *)(s + 16 * nblk) + (uint64_t)r * (K / 32) + u));
    return x;
  }
  template <int M>
  __device__ static __forceinline__ void dot(const Raw &x, uint32_t K, uint32_t u, const uint8_t *acts, uint32_t stride, float *acc, uint32_t n) {
    uint4 lo, hi;
    iq4_lookup8(x.q.x, lo.x, hi.x), iq4_lookup8(x.q.y, lo.y, hi.y), iq4_lookup8(x.q.z, lo.z, hi.z), iq4_lookup8(x.q.w, lo.w, hi.w);
#pragma unroll
    for (int t = 0; t < M; t++) {
      if ((uint32_t)t >= n) break;  // the group's rows: the same for the whole CTA
      const uint8_t *a = acts + t * stride;
      const int4 *av = (const int4 *)(a + 32u * u);
      const int s = dot4x4(lo, av[0]) + dot4x4(hi, av[1]);
      acc[t] = fmaf(x.d * ((const float *)(a + K))[u], (float)s, acc[t]);
    }
  }
};

// IQ4_XS: y = d * (ls - 32) * table[q], 256 values in eight sub-blocks of 32, each with a 6-bit ls: its low four bits
// a nibble of scales_l, its high two a pair of bits of scales_h (QUANT_FORMATS.md:213-232). A unit is one sub-block,
// 16 bytes of qs laid out as IQ4_NL's. Activations are q8_K (its sums are not needed: the table has no offset).
template <>
struct Unit<QT_IQ4_XS> {
  static constexpr int kValues = 32;
  struct Raw {
    uint4 q;
    uint32_t sl, sh;
    float d;
  };
  __device__ static __forceinline__ Raw fetch(const uint8_t *s, uint64_t nblk, uint32_t K, uint32_t r, uint32_t u, const uint32_t *) {
    Raw x;
    x.q = ldg_stream16(s + (uint64_t)r * (K / 2) + 16u * u);
    const uint64_t blk = (uint64_t)r * (K / 256) + u / 8;
    x.sl = __ldg((const uint32_t *)(s + 128 * nblk) + blk);
    x.sh = __ldg((const uint16_t *)(s + 132 * nblk) + blk);
    x.d = __half2float(__ldg((const __half *)(s + 134 * nblk) + blk));
    return x;
  }
  template <int M>
  __device__ static __forceinline__ void dot(const Raw &x, uint32_t K, uint32_t u, const uint8_t *acts, uint32_t stride, float *acc, uint32_t n) {
    const uint32_t b = u / 8, ib = u % 8;
    const int ls = (int)(((x.sl >> (4 * ib)) & 0xF) | (((x.sh >> (2 * ib)) & 3) << 4)) - 32;
    uint4 lo, hi;
    iq4_lookup8(x.q.x, lo.x, hi.x), iq4_lookup8(x.q.y, lo.y, hi.y), iq4_lookup8(x.q.z, lo.z, hi.z), iq4_lookup8(x.q.w, lo.w, hi.w);
#pragma unroll
    for (int t = 0; t < M; t++) {
      if ((uint32_t)t >= n) break;  // the group's rows: the same for the whole CTA
      const uint8_t *a = acts + t * stride;
      const int4 *av = (const int4 *)(a + 256 * b + 32 * ib);
      const int s = dot4x4(lo, av[0]) + dot4x4(hi, av[1]);
      acc[t] = fmaf(x.d * ((const float *)(a + K))[b], (float)(ls * s), acc[t]);
    }
  }
};

template <int QT, int M>
__device__ __forceinline__ void unit_dot(const typename Unit<QT>::Raw &x, uint32_t K, uint32_t u, const uint8_t *acts, uint32_t stride,
                                         float *acc, uint32_t n, const uint32_t *grid) {
  if constexpr (grid_words(QT) > 0)
    Unit<QT>::template dot<M>(x, K, u, acts, stride, acc, n, grid);
  else
    Unit<QT>::template dot<M>(x, K, u, acts, stride, acc, n);
}

// Where the 16-byte piece i of an activation row's codes sits in shared memory. The codebook types' units read four pieces 64 bytes
// apart from lane to lane, which without a swizzle puts a quarter-warp on two groups of four banks (four wavefronts an
// access instead of one): piece (i & 3) of unit i / 4 is stored at (i & 3) ^ ((unit >> 1) & 3).
template <int QT>
__device__ __forceinline__ uint32_t act_slot(uint32_t i) {
  if constexpr (grid_words(QT) > 0) return (i & ~3u) | ((i & 3u) ^ ((i >> 3) & 3u));
  return i;
}

// 16-byte loads a lane keeps in flight: with 8 the Q8_0 kernels fit three CTAs on an SM (16 took 114 registers, two CTAs),
// measured 2 to 5 % faster on steps of 1 to 32 rows.
constexpr int kRowsInFlight = 8;

// Passes of a warp whose loads are issued together: about kRowsInFlight loads of 16 bytes a lane, fewer when many activation rows
// already fill the registers with accumulators.
__host__ __device__ constexpr int rows_batch(int nmat, int nu, int m, bool heavy) {
  // heavy: a unit that holds many registers while it waits (IQ3_S: quants, signs, high bits, scale): fewer passes at
  // once leave room for more CTAs on the SM (three with one pass of gate and up, measured faster than two passes; two
  // passes for the down product, measured faster than one), which its arithmetic-bound decode needs more than loads
  // in flight.
  const int want = kRowsInFlight / (nmat * nu) > 0 ? kRowsInFlight / (nmat * nu) : 1, cap = heavy ? (nmat == 2 ? 1 : 2) : m >= 4 ? 4 : 8;
  return want < cap ? want : cap;
}

// NMAT 2: h[row][r] = swiglu(gate_r . x, up_r . x); NMAT 1: y[row][r] = down_r . h. One CTA of 8 warps per (row tile,
// group); G lanes share a weight row (G = the row's units, up to 32), each taking UPL of its units (UPL 0: as many as
// the row has, found at run time). Launch: grid (R / rows_per_cta, groups at most), 256 threads, dynamic shared memory
// M * act_row_stride (+ 2 KB for IQ3_S's codebook).
template <int QT, int NMAT, int M, int G, int UPL>
__global__ void __launch_bounds__(256) k_expert_rows(const ExpertRowsArgs a, const uint32_t *__restrict__ grid_global) {
  extern __shared__ __align__(16) uint8_t smem[];
  dependents_may_launch(), wait_for_predecessors();
  constexpr bool q8k = act_is_q8k(QT);
  uint32_t slot, start, n;
  if (a.groups) {
    // Both loads go out together: the list is as long as the grid, so the entry can be read before the count says
    // whether it is one (a CTA's life is a chain of dependent loads; this takes one link out).
    const uint32_t ng = __ldg(a.ngroups);
    const MoeGroup g = a.groups[blockIdx.y];
    if (blockIdx.y >= ng) return;
    slot = g.slot, start = g.start, n = g.n;
  } else {
    start = blockIdx.y * M;
    if (start >= a.dense_rows) return;
    slot = 0, n = min((uint32_t)M, a.dense_rows - start);
  }
  const uint32_t K = a.K, stride = act_row_stride(q8k, K), dsz = act_d_bytes(q8k, K);
  const uint32_t upr = K / Unit<QT>::kValues;  // units per weight row
  const uint64_t nblk = (uint64_t)a.R * (K / block_values(QT));
  const uint8_t *w0 = a.w0 + (uint64_t)slot * a.slice_bytes;
  const uint8_t *w1 = NMAT == 2 ? a.w1 + (uint64_t)slot * a.slice_bytes : nullptr;
  const uint32_t warp = threadIdx.x / 32, lane = threadIdx.x % 32, li = lane % G, sub = lane / G;
  constexpr uint32_t RPP = 32 / G;  // weight rows a warp takes per pass
  constexpr int NU = UPL > 0 ? UPL : 1;
  constexpr int RB = rows_batch(NMAT, NU, M, grid_words(QT) > 0);  // passes whose loads go out together
  using Raw = typename Unit<QT>::Raw;
  const uint32_t rows_per_warp = UPL > 0 ? RPP * RB : a.rows_per_cta / 8;
  // A CTA takes `slabs` slabs of 8 * rows_per_warp weight rows one after another, so that what it does once (being
  // launched, finding its group, staging the activations) is spread over more weight bytes.
  const uint32_t slabs = UPL > 0 && a.slabs > 1 ? a.slabs : 1, slab_rows = 8 * rows_per_warp;
  const uint32_t r_begin = blockIdx.x * slabs * slab_rows + warp * rows_per_warp;

  // With the row length known at compile time, every load of the warp's rows goes out first, before the activations
  // are staged: the weights come from HBM and their latency is the kernel's, so as many bytes as the registers hold
  // are put in flight at once.
  Raw raw[RB][NMAT][NU];
  auto fetch_slab = [&](uint32_t base) {
#pragma unroll
    for (int b = 0; b < RB; b++) {
      const uint32_t r = base + b * RPP + sub;
      if (r < a.R) {
#pragma unroll
        for (int j = 0; j < NU; j++) {
          raw[b][0][j] = Unit<QT>::fetch(w0, nblk, K, r, li + G * j, nullptr);
          if constexpr (NMAT == 2) raw[b][1][j] = Unit<QT>::fetch(w1, nblk, K, r, li + G * j, nullptr);
        }
      }
    }
  };
  if constexpr (UPL > 0) fetch_slab(r_begin);

  uint32_t *grid = (uint32_t *)(smem + M * stride);
  if constexpr (grid_words(QT) > 0)
    for (uint32_t i = threadIdx.x; i < grid_words(QT); i += 256) grid[i] = grid_global[grid_offset(QT) + i];
  // The group's activation rows into shared memory; rows past n get zero scales, so they add nothing.
  for (uint32_t t = 0; t < (uint32_t)M; t++) {
    uint8_t *dst = smem + t * stride;
    if (t < n) {
      const uint64_t row = a.act_row ? a.act_row[start + t] : start + t;
      const int4 *src = (const int4 *)(a.act.q + row * a.act.q_stride);
      const float *sd = (const float *)((const uint8_t *)a.act.d + row * a.act.d_stride);
      for (uint32_t i = threadIdx.x; i < K / 16; i += 256) ((int4 *)dst)[act_slot<QT>(i)] = src[i];
      if (q8k) {
        const int16_t *sb = (const int16_t *)((const uint8_t *)a.act.bs + row * a.act.bs_stride);
        for (uint32_t i = threadIdx.x; i < K / 256; i += 256) ((float *)(dst + K))[i] = sd[i];
        for (uint32_t i = threadIdx.x; i < K / 16; i += 256) ((int16_t *)(dst + K + dsz))[i] = sb[i];
      } else {
        for (uint32_t i = threadIdx.x; i < K / 32; i += 256) ((float *)(dst + K))[i] = sd[i];
      }
    } else {
      for (uint32_t i = threadIdx.x; i < dsz / 4; i += 256) ((float *)(dst + K))[i] = 0.0f;
    }
  }
  __syncthreads();

  auto finish = [&](float (&acc)[NMAT][M], uint32_t r) {
#pragma unroll
    for (int m = 0; m < NMAT; m++)
#pragma unroll
      for (int t = 0; t < M; t++)
#pragma unroll
        for (int off = G / 2; off > 0; off >>= 1) acc[m][t] += __shfl_xor_sync(0xffffffffu, acc[m][t], off);
    if (li == 0 && r < a.R) {
#pragma unroll
      for (int t = 0; t < M; t++)
        if ((uint32_t)t < n) {
          float v = acc[0][t];
          if constexpr (NMAT == 2) v = swiglu(acc[0][t], acc[1][t], a.limit);
          a.out[(uint64_t)(start + t) * a.out_stride + r] = v;
        }
    }
  };

  if constexpr (UPL > 0) {
    for (uint32_t sl = 0; sl < slabs; sl++) {
      const uint32_t base = r_begin + sl * slab_rows;
      if (sl > 0) fetch_slab(base);
#pragma unroll
      for (int b = 0; b < RB; b++) {
        const uint32_t r = base + b * RPP + sub;
        float acc[NMAT][M];
#pragma unroll
        for (int m = 0; m < NMAT; m++)
#pragma unroll
          for (int t = 0; t < M; t++) acc[m][t] = 0.0f;
        if (r < a.R) {
#pragma unroll
          for (int j = 0; j < NU; j++) {
            unit_dot<QT, M>(raw[b][0][j], K, li + G * j, smem, stride, acc[0], n, grid);
            if constexpr (NMAT == 2) unit_dot<QT, M>(raw[b][1][j], K, li + G * j, smem, stride, acc[1], n, grid);
          }
        }
        finish(acc, r);
      }
    }
  } else {
    for (uint32_t rr = 0; rr < rows_per_warp; rr += RPP) {
      const uint32_t r = r_begin + rr + sub;
      float acc[NMAT][M];
#pragma unroll
      for (int m = 0; m < NMAT; m++)
#pragma unroll
        for (int t = 0; t < M; t++) acc[m][t] = 0.0f;
      if (r < a.R) {
        for (uint32_t u = li; u < upr; u += G) {
          const Raw x0 = Unit<QT>::fetch(w0, nblk, K, r, u, nullptr);
          unit_dot<QT, M>(x0, K, u, smem, stride, acc[0], n, grid);
          if constexpr (NMAT == 2) {
            const Raw x1 = Unit<QT>::fetch(w1, nblk, K, r, u, nullptr);
            unit_dot<QT, M>(x1, K, u, smem, stride, acc[1], n, grid);
          }
        }
      }
      finish(acc, r);
    }
  }
}

// Launches the instantiation for (M, K): host side of the kernels above. Returns cudaErrorInvalidValue for a shape no
// instantiation takes. max_groups: the grid's second extent.
template <int QT, int NMAT>
cudaError_t launch_expert_rows(const ExpertRowsArgs &a, int M, uint32_t max_groups, const uint32_t *grid_global, cudaStream_t st);

}  // namespace moe
