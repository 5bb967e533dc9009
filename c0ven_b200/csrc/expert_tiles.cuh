// The experts' products for many rows per expert: a grouped GEMM on the 5th-generation tensor cores. A CTA takes 128
// weight rows of one expert and up to 256 of the rows routed to it. Its worker warps decode the quantised blocks to
// f16 straight into shared memory in the tensor core's K-major core-matrix layout and gather the rows' activations
// beside them; one thread issues tcgen05.mma with the weights as the M side and the rows as the N side (so a short
// tile costs a short instruction), accumulating f32 in tensor memory; the workers read the accumulators back with
// tcgen05.ld, apply SwiGLU and store. This replaces the reference's moe_gate_up_t / moe_down_t
// (kernels/quant/qgemm.cl:88-239), whose tiles are 64 rows on Xe2's DPAS.
//
// Operands are IEEE f16, not bf16: the rows are the activations as the CPU path quantises them (q8_0 or q8_K,
// core/cpu/experts.cpp:166-168,229-237), dequantised; with f16's 11-bit significand the products stay within a few
// 1e-3 of that path's integer arithmetic, which bf16's 8 bits do not.
//
// Every wait on an mbarrier is bounded: a wait that runs out raises the CTA's abort flag and a global error word, the
// other waits return at once, and the CTA still frees its tensor memory before it exits.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdint>

#include "expert_rows.cuh"
#include "formats.h"

namespace moe {

// Rows start .. start + count of the expert order, all of one expert; count <= kTileN.
struct BigTile {
  uint32_t slot, start, count;
};
constexpr uint32_t kTileM = 128;   // weight rows a CTA takes
constexpr uint32_t kTileN = 256;   // activation rows at most
constexpr uint32_t kTileK = 64;    // values of the contraction a stage holds
constexpr uint32_t kTileWorkers = 256;

struct ExpertTilesArgs {
  const uint8_t *w0, *w1;   // slot 0's slice of (gate, up) or (down, unused), runs layout
  uint64_t slice_bytes;
  uint32_t K, R;            // values per weight row; weight rows
  const __half *act;        // activation rows, f16 [rows][K]
  const uint32_t *act_row;  // expert-order row -> activation row; null: the same row
  const BigTile *tiles;     // null: dense_rows rows of slot 0 in tiles of kTileN
  const uint32_t *ntiles;
  uint32_t dense_rows;
  float *out;               // out[expert-order row][r], f32
  uint32_t out_stride;
  float limit;
  uint32_t *error;          // set non-zero when a wait ran out
};

namespace tc {

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_test(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// Waits for the barrier's phase `parity` to complete, for about a second at most. False when it gave up or another
// thread of the CTA already had.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile uint32_t *abort, uint32_t *error) {
  if (mbar_test(bar, parity)) return true;
  const long long t0 = clock64();
  for (uint32_t spins = 0;; spins++) {
    if (mbar_test(bar, parity)) return true;
    if (*abort) return false;
    if ((spins & 63) == 63) {
      __nanosleep(64);
      if (clock64() - t0 > 2000000000ll) {
        *abort = 1;
        atomicExch(error, 1u);
        return false;
      }
    }
  }
}
// The arrival happens when every cp.async this thread issued before it has landed; it counts as one of the barrier's
// expected arrivals.
__device__ __forceinline__ void mbar_arrive_after_copies(uint32_t bar) {
  asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void copy_async16(uint32_t dst_smem, const void *src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst_smem), "l"(src) : "memory");
}
__device__ __forceinline__ void fence_barrier_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(ncols) : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_free(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void mma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// D[tmem] (+)= A[smem] * B[smem]^T, f16 operands, f32 accumulate, M 128, K 16.
__device__ __forceinline__ void mma_f16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t *v) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]), "=r"(v[9]),
        "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// A K-major operand tile without swizzle: core matrices of 8 rows x 16 bytes, contiguous (128 bytes); the next 8
// values of the contraction 128 bytes on (the leading offset), the next 8 rows 1024 bytes on (the stride offset).
// Element (row, k) of a stage, k < 64: (row / 8) * 1024 + (k / 8) * 128 + (row % 8) * 16 + (k % 8) * 2.
constexpr uint32_t kLbo = 128, kSbo = 1024;
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr) {
  return (uint64_t)((addr & 0x3FFFFu) >> 4) | ((uint64_t)(kLbo >> 4) << 16) | ((uint64_t)(kSbo >> 4) << 32) | (1ull << 46);
}
// kind::f16 instruction descriptor: f32 accumulator, f16 A and B, both K-major, M 128, N n.
__device__ __forceinline__ uint32_t instr_desc(uint32_t n) { return (1u << 4) | ((n >> 3) << 17) | ((kTileM >> 4) << 24); }

__device__ __forceinline__ void store_chunk(uint8_t *tile, uint32_t row, uint32_t kc, uint4 v) {
  *(uint4 *)(tile + (row >> 3) * kSbo + kc * kLbo + (row & 7) * 16) = v;
}

// Two bytes of x as f16 values 1024 + byte: the exponent byte 0x64 beside each.
__device__ __forceinline__ uint32_t bias_h2(uint32_t x, uint32_t sel) { return __byte_perm(x, 0x64646464u, sel); }
__device__ __forceinline__ __half2 as_h2(uint32_t u) { return *reinterpret_cast<__half2 *>(&u); }
__device__ __forceinline__ uint32_t as_u32(__half2 h) { return *reinterpret_cast<uint32_t *>(&h); }

__device__ __forceinline__ uint4 ldg16(const void *p) {
  uint4 v;
  asm volatile("ld.global.nc.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}

// ---------------------------------------------------------------------------------------------------------------
// Decoders: a stage is 64 values of every one of the tile's 128 weight rows. Decoder<QT>::kUnits units cover it; unit
// i is fetched into registers (Raw) and then written as f16 into the operand tile.
template <int QT>
struct Decoder;

// Q8_0: w = d * q. Unit: 16 codes of a row. 4 units a row.
template <>
struct Decoder<QT_Q8_0> {
  static constexpr uint32_t kUnits = kTileM * 4;
  struct Raw {
    uint4 q;
    __half d;
  };
  __device__ static __forceinline__ Raw fetch(const uint8_t *s, uint64_t nblk, uint32_t K, uint32_t r0, uint32_t k0, uint32_t i) {
    const uint32_t m = (i & 7) | ((i >> 5) << 3), u = (i >> 3) & 3, r = r0 + m;
    Raw x;
    x.q = ldg16(s + (uint64_t)r * K + k0 + 16 * u);
    x.d = __ldg((const __half *)(s + 32 * nblk) + (uint64_t)r * (K / 32) + k0 / 32 + u / 2);
    return x;
  }
  __device__ static __forceinline__ void store(const Raw &x, uint8_t *tile, uint32_t i, const uint32_t *) {
    const uint32_t m = (i & 7) | ((i >> 5) << 3), u = (i >> 3) & 3;
    const __half2 d2 = __half2half2(x.d), off = __float2half2_rn(1152.0f);
    const uint32_t w[4] = {x.q.x ^ 0x80808080u, x.q.y ^ 0x80808080u, x.q.z ^ 0x80808080u, x.q.w ^ 0x80808080u};
    uint32_t h[8];
#pragma unroll
    for (int j = 0; j < 4; j++) {
      h[2 * j] = as_u32(__hmul2(__hsub2(as_h2(bias_h2(w[j], 0x4140)), off), d2));
      h[2 * j + 1] = as_u32(__hmul2(__hsub2(as_h2(bias_h2(w[j], 0x4342)), off), d2));
    }
    store_chunk(tile, m, 2 * u, make_uint4(h[0], h[1], h[2], h[3]));
    store_chunk(tile, m, 2 * u + 1, make_uint4(h[4], h[5], h[6], h[7]));
  }
};

// Q4_K: w = d * sc * q - dmin * m. Unit: 16 bytes of qs, the low nibbles 16 values of sub-block 2c, the high nibbles
// 16 of sub-block 2c + 1, 32 values further on. 2 units a row.
template <>
struct Decoder<QT_Q4_K> {
  static constexpr uint32_t kUnits = kTileM * 2;
  struct Raw {
    uint4 q;
    uint32_t s0, s1, s2;
    __half2 dm;
  };
  __device__ static __forceinline__ Raw fetch(const uint8_t *s, uint64_t nblk, uint32_t K, uint32_t r0, uint32_t k0, uint32_t i) {
    const uint32_t m = (i & 7) | ((i >> 4) << 3), hf = (i >> 3) & 1, r = r0 + m;
    Raw x;
    x.q = ldg16(s + (uint64_t)r * (K / 2) + (k0 / 64) * 32 + 16 * hf);
    const uint64_t blk = (uint64_t)r * (K / 256) + k0 / 256;
    const uint32_t *sc = (const uint32_t *)(s + 128 * nblk + 12 * blk);
    x.s0 = __ldg(sc), x.s1 = __ldg(sc + 1), x.s2 = __ldg(sc + 2);
    x.dm = __ldg((const __half2 *)(s + 140 * nblk + 4 * blk));
    return x;
  }
  __device__ static __forceinline__ uint32_t byte_of(const Raw &x, int i) {
    const uint32_t w = i < 4 ? x.s0 : i < 8 ? x.s1 : x.s2;
    return (w >> (8 * (i & 3))) & 0xFF;
  }
  __device__ static __forceinline__ void scale_min(const Raw &x, int j, int &sc, int &mn) {
    if (j < 4) {
      sc = byte_of(x, j) & 63;
      mn = byte_of(x, j + 4) & 63;
    } else {
      sc = (byte_of(x, j + 4) & 0xF) | ((byte_of(x, j - 4) >> 6) << 4);
      mn = (byte_of(x, j + 4) >> 4) | ((byte_of(x, j) >> 6) << 4);
    }
  }
  __device__ static __forceinline__ void store(const Raw &x, uint8_t *tile, uint32_t i, const uint32_t *, uint32_t k0) {
    const uint32_t m = (i & 7) | ((i >> 4) << 3), hf = (i >> 3) & 1, c = (k0 % 256) / 64;
    int sc_lo, m_lo, sc_hi, m_hi;
    scale_min(x, 2 * c, sc_lo, m_lo);
    scale_min(x, 2 * c + 1, sc_hi, m_hi);
    const float dmin = __high2float(x.dm);
    const __half2 d2 = __half2half2(__low2half(x.dm));
    // (1024 + q) * sc - 1024 * sc = q * sc, exact in f16; then * d - dmin * m, rounded once.
    const __half2 scl = __float2half2_rn((float)sc_lo), sch = __float2half2_rn((float)sc_hi);
    const __half2 bl = __float2half2_rn(-1024.0f * sc_lo), bh = __float2half2_rn(-1024.0f * sc_hi);
    const __half2 ml = __float2half2_rn(-dmin * m_lo), mh = __float2half2_rn(-dmin * m_hi);
    const uint32_t w[4] = {x.q.x, x.q.y, x.q.z, x.q.w};
    uint32_t lo[8], hi[8];
#pragma unroll
    for (int j = 0; j < 4; j++) {
      const uint32_t l = w[j] & 0x0F0F0F0Fu, h = (w[j] >> 4) & 0x0F0F0F0Fu;
      lo[2 * j] = as_u32(__hfma2(__hfma2(as_h2(bias_h2(l, 0x4140)), scl, bl), d2, ml));
      lo[2 * j + 1] = as_u32(__hfma2(__hfma2(as_h2(bias_h2(l, 0x4342)), scl, bl), d2, ml));
      hi[2 * j] = as_u32(__hfma2(__hfma2(as_h2(bias_h2(h, 0x4140)), sch, bh), d2, mh));
      hi[2 * j + 1] = as_u32(__hfma2(__hfma2(as_h2(bias_h2(h, 0x4342)), sch, bh), d2, mh));
    }
    store_chunk(tile, m, 2 * hf, make_uint4(lo[0], lo[1], lo[2], lo[3]));
    store_chunk(tile, m, 2 * hf + 1, make_uint4(lo[4], lo[5], lo[6], lo[7]));
    store_chunk(tile, m, 4 + 2 * hf, make_uint4(hi[0], hi[1], hi[2], hi[3]));
    store_chunk(tile, m, 4 + 2 * hf + 1, make_uint4(hi[4], hi[5], hi[6], hi[7]));
  }
};

// Q6_K: w = d * scales[v / 16] * (q - 32). A stage is half of a block's half: its 64 values take one nibble of 64
// bytes of ql and two bits of 32 bytes of qh. Unit: 16 bytes of ql, 16 values. 4 units a row.
template <>
struct Decoder<QT_Q6_K> {
  static constexpr uint32_t kUnits = kTileM * 4;
  struct Raw {
    uint4 ql, qh;
    int sc;
    __half d;
  };
  __device__ static __forceinline__ Raw fetch(const uint8_t *s, uint64_t nblk, uint32_t K, uint32_t r0, uint32_t k0, uint32_t i) {
    const uint32_t m = (i & 7) | ((i >> 5) << 3), u = (i >> 3) & 3, r = r0 + m;
    const uint32_t v0 = k0 % 256, h = v0 / 128;  // the stage starts at value v0 of its block: 0, 64, 128 or 192
    const uint64_t blk = (uint64_t)r * (K / 256) + k0 / 256;
    Raw x;
    x.ql = ldg16(s + 128 * blk + 64 * h + 16 * u);
    x.qh = ldg16(s + 128 * nblk + 64 * blk + 32 * h + 16 * (u & 1));
    x.sc = __ldg((const int8_t *)(s + 192 * nblk + 16 * blk) + v0 / 16 + u);
    x.d = __ldg((const __half *)(s + 208 * nblk) + blk);
    return x;
  }
  __device__ static __forceinline__ void store(const Raw &x, uint8_t *tile, uint32_t i, const uint32_t *, uint32_t k0) {
    const uint32_t m = (i & 7) | ((i >> 5) << 3), u = (i >> 3) & 3;
    const bool high = (k0 % 128) >= 64;  // values 64..127 of the half: the high nibbles, qh's bits 4..7
    const uint32_t sh = (high ? 4 : 0) + (u >= 2 ? 2 : 0);
    const __half2 dsc = __float2half2_rn(__half2float(x.d) * (float)x.sc), off = __float2half2_rn(1056.0f);
    const uint32_t l[4] = {x.ql.x, x.ql.y, x.ql.z, x.ql.w}, hb[4] = {x.qh.x, x.qh.y, x.qh.z, x.qh.w};
    uint32_t o[8];
#pragma unroll
    for (int j = 0; j < 4; j++) {
      const uint32_t q = ((high ? l[j] >> 4 : l[j]) & 0x0F0F0F0Fu) | (((hb[j] >> sh) & 0x03030303u) << 4);
      o[2 * j] = as_u32(__hmul2(__hsub2(as_h2(bias_h2(q, 0x4140)), off), dsc));
      o[2 * j + 1] = as_u32(__hmul2(__hsub2(as_h2(bias_h2(q, 0x4342)), off), dsc));
    }
    store_chunk(tile, m, 2 * u, make_uint4(o[0], o[1], o[2], o[3]));
    store_chunk(tile, m, 2 * u + 1, make_uint4(o[4], o[5], o[6], o[7]));
  }
};

// IQ3_S: w = d * (1 + 2 s) * grid[index][i] * sign. A stage is two sub-blocks of 32. Unit: 8 bytes of qs, one
// sub-block. 2 units a row.
template <>
struct Decoder<QT_IQ3_S> {
  static constexpr uint32_t kUnits = kTileM * 2;
  struct Raw {
    uint2 qs;
    uint32_t sg, qh, sc;
    __half d;
  };
  __device__ static __forceinline__ Raw fetch(const uint8_t *s, uint64_t nblk, uint32_t K, uint32_t r0, uint32_t k0, uint32_t i) {
    const uint32_t m = (i & 7) | ((i >> 4) << 3), sbi = (i >> 3) & 1, r = r0 + m;
    const uint32_t sb = (k0 % 256) / 32 + sbi;  // the sub-block within its block
    const uint64_t blk = (uint64_t)r * (K / 256) + k0 / 256;
    Raw x;
    x.qs = __ldg((const uint2 *)(s + 64 * blk + 8 * sb));
    x.sg = __ldg((const uint32_t *)(s + 64 * nblk + 32 * blk + 4 * sb));
    x.qh = __ldg(s + 96 * nblk + 8 * blk + sb);
    x.sc = (__ldg(s + 104 * nblk + 4 * blk + sb / 2) >> (4 * (sb & 1))) & 0xF;
    x.d = __ldg((const __half *)(s + 108 * nblk) + blk);
    return x;
  }
  __device__ static __forceinline__ void store(const Raw &x, uint8_t *tile, uint32_t i, const uint32_t *grid, uint32_t) {
    const uint32_t m = (i & 7) | ((i >> 4) << 3), sbi = (i >> 3) & 1;
    const __half2 ls = __float2half2_rn((float)(2 * x.sc + 1)), d2 = __half2half2(x.d), off = __float2half2_rn(1024.0f);
    uint32_t o[16];
#pragma unroll
    for (int k = 0; k < 8; k++) {
      const uint32_t word = k < 4 ? x.qs.x : x.qs.y;
      const uint32_t g = grid[((word >> (8 * (k & 3))) & 0xFF) | (((x.qh >> k) & 1u) << 8)];
      const uint32_t nib = (x.sg >> (4 * k)) & 0xF;
      // The sign bit of each f16: values 4k, 4k + 1 from the nibble's bits 0, 1; 4k + 2, 4k + 3 from bits 2, 3.
      const uint32_t s01 = ((nib & 1u) << 15) | ((nib & 2u) << 30), s23 = ((nib & 4u) << 13) | ((nib & 8u) << 28);
      o[2 * k] = as_u32(__hmul2(__hmul2(__hsub2(as_h2(bias_h2(g, 0x4140)), off), ls), d2)) ^ s01;
      o[2 * k + 1] = as_u32(__hmul2(__hmul2(__hsub2(as_h2(bias_h2(g, 0x4342)), off), ls), d2)) ^ s23;
    }
#pragma unroll
    for (int c = 0; c < 4; c++) store_chunk(tile, m, 4 * sbi + c, make_uint4(o[4 * c], o[4 * c + 1], o[4 * c + 2], o[4 * c + 3]));
  }
};

template <int QT>
__device__ __forceinline__ void decode_store(const typename Decoder<QT>::Raw &x, uint8_t *tile, uint32_t i, const uint32_t *grid, uint32_t k0) {
  if constexpr (QT == QT_Q8_0)
    Decoder<QT>::store(x, tile, i, grid);
  else
    Decoder<QT>::store(x, tile, i, grid, k0);
}

}  // namespace tc

// Shared memory of a CTA: the stages (NMAT weight tiles of 16 KB and a row tile of 32 KB each), then the barriers.
template <int NMAT>
struct TileSmem {
  static constexpr uint32_t kStages = NMAT == 2 ? 3 : 4;
  static constexpr uint32_t kWBytes = kTileM * kTileK * 2, kXBytes = kTileN * kTileK * 2;
  static constexpr uint32_t kStageBytes = NMAT * kWBytes + kXBytes;
  static constexpr uint32_t kBarriers = kStages * kStageBytes;  // full[kStages], empty[kStages], acc, then tmem address, abort
  static constexpr uint32_t kGrid = kBarriers + 128;            // IQ3_S's codebook, 2 KB
  static constexpr uint32_t kRowIdx = kGrid + 2048;             // the tile's activation rows, kTileN words
  static constexpr uint32_t kBytes = kRowIdx + 4 * kTileN + 1024;  // and room to align the base to 1024
};

// NMAT 2: out = swiglu(gate x, up x); NMAT 1: out = down h. Launch: grid (R / 128, tiles at most), 288 threads
// (8 worker warps, then the warp that owns tensor memory and issues the MMAs), dynamic shared memory TileSmem::kBytes.
template <int QT, int NMAT>
__global__ void __launch_bounds__(288, 1) k_expert_tiles(const ExpertTilesArgs a, const uint32_t *__restrict__ grid_global) {
  using namespace tc;
  using SM = TileSmem<NMAT>;
  using Dec = Decoder<QT>;
  constexpr uint32_t S = SM::kStages;
  extern __shared__ uint8_t smem_raw[];
  uint8_t *smem = (uint8_t *)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);

  uint32_t slot, start, count;
  if (a.tiles) {
    if (blockIdx.y >= *a.ntiles) return;
    const BigTile t = a.tiles[blockIdx.y];
    slot = t.slot, start = t.start, count = t.count;
  } else {
    start = blockIdx.y * kTileN;
    if (start >= a.dense_rows) return;
    slot = 0, count = min(kTileN, a.dense_rows - start);
  }
  const uint32_t K = a.K, KT = K / kTileK, r0 = blockIdx.x * kTileM;
  const uint32_t N = (count + 15) & ~15u;  // the MMA's N: the rows, rounded up to 16
  const uint32_t tid = threadIdx.x, warp = tid / 32, lane = tid % 32;
  uint64_t *bars = (uint64_t *)(smem + SM::kBarriers);
  const uint32_t bar0 = smem_u32(bars);
  auto full_bar = [&](uint32_t s) { return bar0 + 8 * s; };
  auto empty_bar = [&](uint32_t s) { return bar0 + 8 * (S + s); };
  const uint32_t acc_bar = bar0 + 8 * (2 * S);
  uint32_t *tmem_slot = (uint32_t *)(bars + 2 * S + 1);
  volatile uint32_t *abort = tmem_slot + 1;
  uint32_t *grid = (uint32_t *)(smem + SM::kGrid);
  uint32_t *rowidx = (uint32_t *)(smem + SM::kRowIdx);
  constexpr uint32_t kCols = NMAT == 2 ? 512 : 256;

  // A stage is full when every worker has stored its decoded weights (one arrival) and its copies of the rows'
  // activations have landed (one more, made by the copy unit).
  if (tid == 0) {
    for (uint32_t s = 0; s < S; s++) mbar_init(full_bar(s), 2 * kTileWorkers), mbar_init(empty_bar(s), 1);
    mbar_init(acc_bar, 1);
    *abort = 0;
    fence_barrier_init();
  }
  if constexpr (QT == QT_IQ3_S)
    for (uint32_t i = tid; i < 512; i += blockDim.x) grid[i] = grid_global[i];
  for (uint32_t n = tid; n < kTileN; n += blockDim.x)
    rowidx[n] = n < count ? (a.act_row ? a.act_row[start + n] : start + n) : 0xFFFFFFFFu;
  if (warp == 8) tmem_alloc(smem_u32(tmem_slot), kCols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp < 8) {
    // Workers: decode this stage's weights and gather its rows' activations into the operand tiles.
    const uint64_t nblk = (uint64_t)a.R * (K / block_values(QT));
    const uint8_t *w0 = a.w0 + (uint64_t)slot * a.slice_bytes;
    const uint8_t *w1 = NMAT == 2 ? a.w1 + (uint64_t)slot * a.slice_bytes : nullptr;
    constexpr uint32_t UPT = Dec::kUnits / kTileWorkers;  // weight units a thread takes per matrix and stage
    using Raw = typename Dec::Raw;
    const uint32_t nchunks = N * 8;  // 16-byte pieces of the rows' activations in a stage
    bool ok = true;
    Raw raw[2][NMAT][UPT];  // this stage's quants and the next one's, fetched a stage ahead
    auto fetch = [&](Raw (&r)[NMAT][UPT], uint32_t k0) {
#pragma unroll
      for (uint32_t j = 0; j < UPT; j++) {
        r[0][j] = Dec::fetch(w0, nblk, K, r0, k0, tid + j * kTileWorkers);
        if constexpr (NMAT == 2) r[1][j] = Dec::fetch(w1, nblk, K, r0, k0, tid + j * kTileWorkers);
      }
    };
    auto stage_step = [&](Raw (&r)[NMAT][UPT], uint32_t it) {
      const uint32_t s = it % S, k0 = it * kTileK;
      uint8_t *stage = smem + s * SM::kStageBytes;
      if (it >= S) ok = mbar_wait(empty_bar(s), ((it / S) - 1) & 1, abort, a.error);
      if (!ok) return;
      tc_fence_after();
      // The rows' activations: 16-byte asynchronous copies by token index, straight into the operand layout. Piece c
      // is (row n, chunk kc); 8 consecutive threads take the 8 rows of a core matrix. Rows past count are never read
      // back (their columns of the result are dropped), so they are left as they are.
      const uint32_t xt = smem_u32(stage + NMAT * SM::kWBytes);
      for (uint32_t c = tid; c < nchunks; c += kTileWorkers) {
        const uint32_t n = (c & 7) | ((c >> 6) << 3), kc = (c >> 3) & 7, row = rowidx[n];
        if (row != 0xFFFFFFFFu) copy_async16(xt + (n >> 3) * kSbo + kc * kLbo + (n & 7) * 16, a.act + (uint64_t)row * K + k0 + 8 * kc);
      }
      mbar_arrive_after_copies(full_bar(s));
#pragma unroll
      for (uint32_t j = 0; j < UPT; j++) {
        decode_store<QT>(r[0][j], stage, tid + j * kTileWorkers, grid, k0);
        if constexpr (NMAT == 2) decode_store<QT>(r[1][j], stage + SM::kWBytes, tid + j * kTileWorkers, grid, k0);
      }
      fence_async_smem();
      mbar_arrive(full_bar(s));
    };
    fetch(raw[0], 0);
    for (uint32_t it = 0; it < KT && ok; it += 2) {
      if (it + 1 < KT) fetch(raw[1], (it + 1) * kTileK);
      stage_step(raw[0], it);
      if (!ok || it + 1 >= KT) break;
      if (it + 2 < KT) fetch(raw[0], (it + 2) * kTileK);
      stage_step(raw[1], it + 1);
    }
    // Epilogue: warp w reads TMEM lanes 32 (w % 4) .., its row of the weights; warps w and w + 4 share the columns.
    if (ok) ok = mbar_wait(acc_bar, 0, abort, a.error);
    if (ok) {
      tc_fence_after();
      const uint32_t q = warp % 4, r = r0 + 32 * q + lane;
      for (uint32_t c = warp / 4; c < N / 16; c += 2) {
        uint32_t g[16], u[16];
        tmem_ld16(tmem_base + ((32 * q) << 16) + 16 * c, g);
        if constexpr (NMAT == 2) tmem_ld16(tmem_base + ((32 * q) << 16) + kTileN + 16 * c, u);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 16; j++) {
          const uint32_t n = 16 * c + j;
          if (n < count && r < a.R) {
            float v = __uint_as_float(g[j]);
            if constexpr (NMAT == 2) v = swiglu(v, __uint_as_float(u[j]), a.limit);
            a.out[(uint64_t)(start + n) * a.out_stride + r] = v;
          }
        }
      }
    }
  } else if (lane == 0) {
    // The MMA thread: per stage, four K steps of 16 for each matrix; the commit frees the stage when they are done.
    const uint32_t idesc = instr_desc(N);
    bool ok = true;
    for (uint32_t it = 0; it < KT && ok; it++) {
      const uint32_t s = it % S;
      ok = mbar_wait(full_bar(s), (it / S) & 1, abort, a.error);
      if (!ok) break;
      fence_async_smem();  // the copies' writes, like the workers' stores, must be visible to the tensor core's reads
      tc_fence_after();
      const uint32_t stage = smem_u32(smem + s * SM::kStageBytes), xt = stage + NMAT * SM::kWBytes;
#pragma unroll
      for (uint32_t k = 0; k < kTileK / 16; k++) {
        const uint64_t db = smem_desc(xt + 2 * k * kLbo);
        mma_f16(tmem_base, smem_desc(stage + 2 * k * kLbo), db, idesc, (it | k) != 0);
        if constexpr (NMAT == 2) mma_f16(tmem_base + kTileN, smem_desc(stage + SM::kWBytes + 2 * k * kLbo), db, idesc, (it | k) != 0);
      }
      mma_commit(empty_bar(s));
    }
    if (ok) mma_commit(acc_bar);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 8) {
    __syncwarp();
    tc_fence_after();
    tmem_free(tmem_base, kCols);
  }
}

template <int QT, int NMAT>
cudaError_t launch_expert_tiles(const ExpertTilesArgs &a, uint32_t max_tiles, const uint32_t *grid_global, cudaStream_t st);

}  // namespace moe
