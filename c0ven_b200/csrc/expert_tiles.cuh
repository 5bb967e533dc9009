// The experts' products for many rows per expert: a grouped GEMM on the 5th-generation tensor cores. A work item is 128
// weight rows of one expert and up to 256 of the rows routed to it; persistent CTAs, one per SM, take items in turn.
// Decode warps turn the quantised blocks into f16 straight into shared memory in the tensor core's K-major
// core-matrix layout; one thread brings the rows' activations beside them with bulk-tensor (TMA) copies, 64 rows a
// copy, in the 128-byte-swizzled K-major layout; one thread issues tcgen05.mma with the weights as the M side and the rows as the N side (so a short
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

#include <cuda.h>
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
constexpr uint32_t kTileDecoders = 512;  // threads that decode weights: 16 warps, enough of them to hide their loads' latency
constexpr uint32_t kTileEpilogue = 128;  // threads that turn accumulators into results: a warp per quarter of the weight rows
constexpr uint32_t kTileThreads = kTileDecoders + kTileEpilogue + 96;  // and the rows' copy warp, the MMA warp, the quants' copy warp
constexpr uint32_t kTileBoxRows = 64;    // rows one bulk-tensor copy brings (the tensor map's box: 64 values x 64 rows)

struct ExpertTilesArgs {
  const uint8_t *w0, *w1;   // slot 0's slice of (gate, up) or (down, unused), runs layout
  uint64_t slice_bytes;
  uint32_t K, R;            // values per weight row; weight rows
                            // the activation rows, f16 [rows][K] in the order of the tiles, come through the tensor map
  const BigTile *tiles;     // null: dense_rows rows of slot 0 in tiles of kTileN
  const uint32_t *ntiles;
  uint32_t dense_rows;
  const uint32_t *gather_rows;  // not null: row r of the tiles' order is row gather_rows[r] of the map's tensor, whose box is
                                // one row (the copies gather four rows each); null: the same row, boxes of 64 rows
  void *out;                // out[expert-order row][r]: f32, or f16 when out_f16 is set
  uint32_t out_stride;
  uint32_t out_f16;
  float limit;
  uint32_t *error;          // set non-zero when a wait ran out
  // For types whose quants come by copy (quants_by_copy): maps over the quants runs of w0 and w1, (bytes of a row, rows,
  // expert slots), their box (a quant slot's bytes a row, 128 rows, 1 slot) (tensor_map.h: make_quants_map).
  CUtensorMap qmap[2];
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
// One bounded hardware wait: the warp sleeps until the phase completes or the hint (in ns) runs out.
__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity, uint32_t hint_ns) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity), "r"(hint_ns)
      : "memory");
  return ok != 0;
}
// Waits for the barrier's phase `parity` to complete, for about a second at most. False when it gave up or another
// thread of the CTA already had. The wait suspends the warp rather than spinning, so it takes no issue slots from the
// warps that decode.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile uint32_t *abort, uint32_t *error) {
  if (mbar_test(bar, parity)) return true;
  const long long t0 = clock64();
  for (;;) {
    if (mbar_try(bar, parity, 20000)) return true;
    if (*abort) return false;
    if (clock64() - t0 > 2000000000ll) {
      *abort = 1;
      atomicExch(error, 1u);
      return false;
    }
  }
}
// One arrival that also tells the barrier to expect `bytes` of bulk copies before its phase completes.
__device__ __forceinline__ void mbar_arrive_expect(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
// Box (x .. x + 63 values, y .. y + 63 rows) of the map's tensor into shared memory at dst (1024-byte aligned); the
// bytes are counted on the barrier as they land. x * 2 bytes is a multiple of 16, as every bulk-tensor copy needs.
__device__ __forceinline__ void tma_load_rows(uint32_t dst_smem, const CUtensorMap *map, uint32_t x, uint32_t y, uint32_t bar) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
               ::"r"(dst_smem), "l"((uint64_t)map), "r"(x), "r"(y), "r"(bar)
               : "memory");
}
// Four rows y0 .. y3 of the map's tensor (its box one row of 64 values), values x .. x + 63 of each, into four
// consecutive 128-byte rows of shared memory at dst (512-byte aligned inside a 1024-byte aligned tile), swizzled as the
// tile's other rows are. The rows need not be neighbours: this is how a tile's rows are gathered by index.
__device__ __forceinline__ void tma_gather4_rows(uint32_t dst_smem, const CUtensorMap *map, uint32_t x, uint32_t y0, uint32_t y1, uint32_t y2,
                                                 uint32_t y3, uint32_t bar) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile::gather4.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5, %6}], [%7];"
               ::"r"(dst_smem), "l"((uint64_t)map), "r"(x), "r"(y0), "r"(y1), "r"(y2), "r"(y3), "r"(bar)
               : "memory");
}
// The same by a CTA of a pair, the bytes counted on a barrier that may be the other CTA's.
__device__ __forceinline__ void tma_gather4_rows_pair(uint32_t dst_smem, const CUtensorMap *map, uint32_t x, uint32_t y0, uint32_t y1,
                                                      uint32_t y2, uint32_t y3, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.tile::gather4.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5, %6}], [%7];"
      ::"r"(dst_smem), "l"((uint64_t)map), "r"(x), "r"(y0), "r"(y1), "r"(y2), "r"(y3), "r"(bar)
      : "memory");
}
// Box (x .. of the row's bytes, rows y .., expert slot z) of a weight matrix's quants run into shared memory at dst.
// x is a multiple of 16 bytes.
__device__ __forceinline__ void tma_load_quants(uint32_t dst_smem, const CUtensorMap *map, uint32_t x, uint32_t y, uint32_t z, uint32_t bar) {
  asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
               ::"r"(dst_smem), "l"((uint64_t)map), "r"(x), "r"(y), "r"(z), "r"(bar)
               : "memory");
}
// --- A pair of CTAs (a cluster of two on the two SMs of a TPC) that share one product: tcgen05's cta_group::2. ---
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// The shared::cluster address of the same place in CTA `rank` of the cluster.
__device__ __forceinline__ uint32_t map_to_cta(uint32_t addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}
// Arrivals on a barrier that may be the other CTA's (a shared::cluster address). What the arriving thread wrote for the
// tensor core to read has passed its own fence.proxy.async before; a release for the whole cluster on every arrival
// was measured to cost the decode warps a third of their rate and is left out, as in CUTLASS's pipelines for a pair.
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_cluster(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cluster.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
// All threads of both CTAs.
__device__ __forceinline__ void cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// tma_load_rows by a CTA of a pair: the bytes land in this CTA's shared memory and are counted on the barrier `bar`,
// which may be the other CTA's (a shared::cluster address).
__device__ __forceinline__ void tma_load_rows_pair(uint32_t dst_smem, const CUtensorMap *map, uint32_t x, uint32_t y, uint32_t bar) {
  asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
               ::"r"(dst_smem), "l"((uint64_t)map), "r"(x), "r"(y), "r"(bar)
               : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t dst_smem, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(ncols) : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_free_pair(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// The pair's commit: one arrival on the barrier at this place in each CTA of the mask.
__device__ __forceinline__ void mma_commit_pair(uint32_t bar, uint32_t cta_mask) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(bar), "h"((uint16_t)cta_mask)
               : "memory");
}
// D[tmem of both CTAs] (+)= A[256 rows: 128 in each CTA's shared memory] * B[n rows: half in each CTA's]^T, issued by
// one thread of the pair's first CTA; the descriptors name the same places in both.
__device__ __forceinline__ void mma_f16_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5, %5, %5, %5, %5}, p;\n\t}"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(0u)
      : "memory");
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
__device__ __forceinline__ void tmem_ld8(uint32_t taddr, uint32_t *v) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
               : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7])
               : "r"(taddr)
               : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
// The wait, naming the registers the loads fill: nothing that reads them can be scheduled before it.
__device__ __forceinline__ void tmem_ld_wait8(uint32_t *v) {
  asm volatile("tcgen05.wait::ld.sync.aligned;"
               : "+r"(v[0]), "+r"(v[1]), "+r"(v[2]), "+r"(v[3]), "+r"(v[4]), "+r"(v[5]), "+r"(v[6]), "+r"(v[7])
               :
               : "memory");
}
__device__ __forceinline__ void tmem_ld_wait16(uint32_t *v) {
  asm volatile("tcgen05.wait::ld.sync.aligned;"
               : "+r"(v[0]), "+r"(v[1]), "+r"(v[2]), "+r"(v[3]), "+r"(v[4]), "+r"(v[5]), "+r"(v[6]), "+r"(v[7]), "+r"(v[8]), "+r"(v[9]),
                 "+r"(v[10]), "+r"(v[11]), "+r"(v[12]), "+r"(v[13]), "+r"(v[14]), "+r"(v[15])
               :
               : "memory");
}

// A K-major operand tile without swizzle: core matrices of 8 rows x 16 bytes, contiguous (128 bytes); the next 8
// values of the contraction 128 bytes on (the leading offset), the next 8 rows 1024 bytes on (the stride offset).
// Element (row, k) of a stage, k < 64: (row / 8) * 1024 + (k / 8) * 128 + (row % 8) * 16 + (k % 8) * 2.
constexpr uint32_t kLbo = 128, kSbo = 1024;
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr) {
  return (uint64_t)((addr & 0x3FFFFu) >> 4) | ((uint64_t)(kLbo >> 4) << 16) | ((uint64_t)(kSbo >> 4) << 32) | (1ull << 46);
}
// The rows' tile as the bulk-tensor copies lay it: a row is 128 contiguous bytes (64 values) whose 16-byte pieces are
// swizzled by the row's low three bits; 8 rows 1024 bytes on. The next 16 values of the contraction: 32 bytes on.
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t addr) {
  return (uint64_t)((addr & 0x3FFFFu) >> 4) | ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
}
// kind::f16 instruction descriptor: f32 accumulator, f16 A and B, both K-major, M 128, N n.
__device__ __forceinline__ uint32_t instr_desc(uint32_t n, uint32_t m = kTileM) { return (1u << 4) | ((n >> 3) << 17) | ((m >> 4) << 24); }

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


__device__ __forceinline__ void prefetch_l2(const void *p) { asm volatile("prefetch.global.L2 [%0];" ::"l"(p)); }

// Small integers as f16 without an int-to-float conversion: 0x6400 | v is 1024 + v for v < 1024.
__device__ __forceinline__ __half2 small_h2(uint32_t v) { return __hsub2(as_h2(0x64006400u | v | (v << 16)), as_h2(0x64006400u)); }

// ---------------------------------------------------------------------------------------------------------------
// Decoders. A stage is 64 values of every one of the tile's 128 weight rows; a thread takes one half of a row's stage,
// 32 values: it fetches the half's quants and scales into registers (Raw), a stage ahead, and later writes them as f16
// into the operand tile, chunks 4 h .. 4 h + 3 of row m. All arithmetic is in f16 pairs; integers reach f16 through
// the exponent trick above, never through a conversion instruction.
template <int QT>
struct Decoder;

// Q8_0: w = d * q. A half is one block.
template <>
struct Decoder<QT_Q8_0> {
  static constexpr uint32_t kStageBytes = 64;  // bytes of a row's main quants run a 64-value stage reads
  struct Hdr {};
  __device__ static __forceinline__ Hdr fetch_hdr(const uint8_t *, uint64_t, uint32_t, uint32_t, uint32_t) { return Hdr{}; }
  struct Raw {
    uint4 q0, q1;
    __half d;
  };
  __device__ static __forceinline__ const uint8_t *quants_at(const uint8_t *s, uint64_t, uint32_t K, uint32_t r, uint32_t k0, uint32_t h) {
    return s + (uint64_t)r * K + k0 + 32 * h;
  }
  __device__ static __forceinline__ Raw fetch(const uint8_t *s, uint64_t nblk, uint32_t K, uint32_t r, uint32_t k0, uint32_t h) {
    Raw x;
    const uint8_t *q = s + (uint64_t)r * K + k0 + 32 * h;
    x.q0 = ldg16(q), x.q1 = ldg16(q + 16);
    x.d = __ldg((const __half *)(s + 32 * nblk) + (uint64_t)r * (K / 32) + k0 / 32 + h);
    return x;
  }
  __device__ static __forceinline__ void store(const Hdr &, const Raw &x, uint8_t *tile, uint32_t m, uint32_t h, uint32_t, const uint32_t *) {
    const __half2 d2 = __half2half2(x.d), off = as_h2(0x64806480u);  // 1152 = 1024 + 128
    const uint32_t w[8] = {x.q0.x, x.q0.y, x.q0.z, x.q0.w, x.q1.x, x.q1.y, x.q1.z, x.q1.w};
    uint32_t o[16];
#pragma unroll
    for (int j = 0; j < 8; j++) {
      const uint32_t u = w[j] ^ 0x80808080u;  // int8 + 128
      o[2 * j] = as_u32(__hmul2(__hsub2(as_h2(bias_h2(u, 0x4140)), off), d2));
      o[2 * j + 1] = as_u32(__hmul2(__hsub2(as_h2(bias_h2(u, 0x4342)), off), d2));
    }
#pragma unroll
    for (int c = 0; c < 4; c++) store_chunk(tile, m, 4 * h + c, make_uint4(o[4 * c], o[4 * c + 1], o[4 * c + 2], o[4 * c + 3]));
  }
};

// Q4_K: w = d * sc * q - dmin * m. A stage is 32 bytes of qs: their low nibbles are its first 32 values (sub-block 2c),
// their high nibbles its second 32 (sub-block 2c + 1). The two threads of a row's stage take 16 of the 32 bytes each,
// both nibbles: values 16 h .. 16 h + 15 of each sub-block, chunks 2 h, 2 h + 1 and 4 + 2 h, 5 + 2 h of the stage. The
// block's d, dmin and scales are one 16-byte piece, loaded once for its four stages.
template <>
struct Decoder<QT_Q4_K> {
  static constexpr uint32_t kStageBytes = 32;  // bytes of a row's main quants run a 64-value stage reads
  struct Hdr {
    uint4 v;  // d, dmin; then the 12 bytes of packed scales and minimums
  };
  struct Raw {
    uint4 q;
  };
  __device__ static __forceinline__ Hdr fetch_hdr(const uint8_t *s, uint64_t nblk, uint32_t K, uint32_t r, uint32_t k0) {
    return Hdr{__ldg((const uint4 *)(s + 128 * nblk + 16 * ((uint64_t)r * (K / 256) + k0 / 256)))};
  }
  __device__ static __forceinline__ const uint8_t *quants_at(const uint8_t *s, uint64_t, uint32_t K, uint32_t r, uint32_t k0, uint32_t h) {
    return s + (uint64_t)r * (K / 2) + (k0 / 64) * 32 + 16 * h;
  }
  __device__ static __forceinline__ Raw fetch(const uint8_t *s, uint64_t nblk, uint32_t K, uint32_t r, uint32_t k0, uint32_t h) {
    return Raw{ldg16(quants_at(s, nblk, K, r, k0, h))};
  }
  // The 6-bit scale and minimum of sub-blocks 2 c and 2 c + 1 (QUANT_FORMATS.md:386-392), each pair as two bytes of a word.
  __device__ static __forceinline__ void scales_of(const Hdr &x, uint32_t c, uint32_t &sc, uint32_t &mn) {
    // Bytes 2 c, 2 c + 1 of the three words of packed scales: words y (bytes 0-3), z (4-7), w (8-11).
    const uint32_t lo = c & 1 ? 0x7732u : 0x7710u;  // byte_perm selector for bytes 2 (c & 1), 2 (c & 1) + 1, zero-extended
    if (c < 2) {
      sc = __byte_perm(x.v.y, 0, lo) & 0x3F3Fu, mn = __byte_perm(x.v.z, 0, lo) & 0x3F3Fu;
    } else {
      const uint32_t p = __byte_perm(x.v.w, 0, lo), a = __byte_perm(x.v.y, 0, lo), b = __byte_perm(x.v.z, 0, lo);
      sc = (p & 0x0F0Fu) | ((a >> 2) & 0x3030u), mn = ((p >> 4) & 0x0F0Fu) | ((b >> 2) & 0x3030u);
    }
  }
  __device__ static __forceinline__ void store(const Hdr &hd, const Raw &x, uint8_t *tile, uint32_t m, uint32_t h, uint32_t k0, const uint32_t *) {
    uint32_t sc, mn;
    scales_of(hd, (k0 % 256) / 64, sc, mn);
    // A byte beside the exponent byte 0x64 is the f16 value 1024 + byte: 1024 + q for a low nibble, 1024 + 16 q for a
    // high nibble left in place. q comes out exactly (v - 1024, or v / 16 - 64 in one fused step); then w = a * q + c
    // with a = d * sc and c = -dmin * m, rounded once.
    const __half2 dm = as_h2(hd.v.x);
    const float d = __low2float(dm), dmin = __high2float(dm);
    const __half2 A0 = __float2half2_rn(d * (float)(sc & 0xFF)), A1 = __float2half2_rn(d * (float)(sc >> 8));
    const __half2 C0 = __float2half2_rn(-dmin * (float)(mn & 0xFF)), C1 = __float2half2_rn(-dmin * (float)(mn >> 8));
    const __half2 k1024 = as_h2(0x64006400u), k16th = as_h2(0x2C002C00u), km64 = as_h2(0xD400D400u);  // 1024, 1/16, -64
    const uint32_t w[4] = {x.q.x, x.q.y, x.q.z, x.q.w};
    uint32_t lo[8], hi[8];
#pragma unroll
    for (int i = 0; i < 4; i++) {
      const uint32_t l = w[i] & 0x0F0F0F0Fu, g = w[i] & 0xF0F0F0F0u;
      lo[2 * i] = as_u32(__hfma2(__hsub2(as_h2(bias_h2(l, 0x4140)), k1024), A0, C0));
      lo[2 * i + 1] = as_u32(__hfma2(__hsub2(as_h2(bias_h2(l, 0x4342)), k1024), A0, C0));
      hi[2 * i] = as_u32(__hfma2(__hfma2(as_h2(bias_h2(g, 0x4140)), k16th, km64), A1, C1));
      hi[2 * i + 1] = as_u32(__hfma2(__hfma2(as_h2(bias_h2(g, 0x4342)), k16th, km64), A1, C1));
    }
    store_chunk(tile, m, 2 * h, make_uint4(lo[0], lo[1], lo[2], lo[3]));
    store_chunk(tile, m, 2 * h + 1, make_uint4(lo[4], lo[5], lo[6], lo[7]));
    store_chunk(tile, m, 4 + 2 * h, make_uint4(hi[0], hi[1], hi[2], hi[3]));
    store_chunk(tile, m, 5 + 2 * h, make_uint4(hi[4], hi[5], hi[6], hi[7]));
  }
};

// Q6_K: w = d * scales[v / 16] * (q - 32). A stage is a quarter of a block: one nibble of 64 bytes of ql and two bits
// of 32 bytes of qh; a half is 32 bytes of ql with all 32 of qh, two groups of 16 with a scale each.
template <>
struct Decoder<QT_Q6_K> {
  static constexpr uint32_t kStageBytes = 32;  // bytes of a row's main quants run a 64-value stage reads
  struct Hdr {};
  __device__ static __forceinline__ Hdr fetch_hdr(const uint8_t *, uint64_t, uint32_t, uint32_t, uint32_t) { return Hdr{}; }
  struct Raw {
    uint4 l0, l1, h0, h1;
    int sc0, sc1;
    __half d;
  };
  __device__ static __forceinline__ const uint8_t *quants_at(const uint8_t *s, uint64_t, uint32_t K, uint32_t r, uint32_t k0, uint32_t h) {
    return s + 128 * ((uint64_t)r * (K / 256) + k0 / 256) + 64 * ((k0 % 256) / 128) + 32 * h;
  }
  __device__ static __forceinline__ Raw fetch(const uint8_t *s, uint64_t nblk, uint32_t K, uint32_t r, uint32_t k0, uint32_t h) {
    const uint32_t v0 = k0 % 256, hh = v0 / 128;  // the stage starts at value v0 of its block: 0, 64, 128 or 192
    const uint64_t blk = (uint64_t)r * (K / 256) + k0 / 256;
    Raw x;
    const uint8_t *ql = s + 128 * blk + 64 * hh + 32 * h, *qh = s + 128 * nblk + 64 * blk + 32 * hh;
    x.l0 = ldg16(ql), x.l1 = ldg16(ql + 16), x.h0 = ldg16(qh), x.h1 = ldg16(qh + 16);
    const int8_t *sc = (const int8_t *)(s + 192 * nblk + 16 * blk) + v0 / 16 + 2 * h;
    x.sc0 = __ldg(sc), x.sc1 = __ldg(sc + 1);
    x.d = __ldg((const __half *)(s + 208 * nblk) + blk);
    return x;
  }
  __device__ static __forceinline__ void store(const Hdr &, const Raw &x, uint8_t *tile, uint32_t m, uint32_t h, uint32_t k0, const uint32_t *) {
    const bool high = (k0 % 128) >= 64;  // values 64 .. 127 of the block's half: the high nibbles, qh's bits 4 .. 7
    const uint32_t sh = (high ? 4 : 0) + (h ? 2 : 0), nsh = high ? 4 : 0;
    const __half2 d2 = __half2half2(x.d), off = as_h2(0x64206420u), o128 = as_h2(0x64806480u);  // 1056 = 1024 + 32; 1152
    const __half2 ds0 = __hmul2(d2, __hsub2(as_h2(0x64006400u | (uint32_t)(x.sc0 + 128) * 0x10001u), o128));
    const __half2 ds1 = __hmul2(d2, __hsub2(as_h2(0x64006400u | (uint32_t)(x.sc1 + 128) * 0x10001u), o128));
    const uint32_t l[8] = {x.l0.x, x.l0.y, x.l0.z, x.l0.w, x.l1.x, x.l1.y, x.l1.z, x.l1.w};
    const uint32_t b[8] = {x.h0.x, x.h0.y, x.h0.z, x.h0.w, x.h1.x, x.h1.y, x.h1.z, x.h1.w};
    uint32_t o[16];
#pragma unroll
    for (int i = 0; i < 8; i++) {
      const uint32_t q = ((l[i] >> nsh) & 0x0F0F0F0Fu) | (((b[i] >> sh) & 0x03030303u) << 4);
      const __half2 ds = i < 4 ? ds0 : ds1;
      o[2 * i] = as_u32(__hmul2(__hsub2(as_h2(bias_h2(q, 0x4140)), off), ds));
      o[2 * i + 1] = as_u32(__hmul2(__hsub2(as_h2(bias_h2(q, 0x4342)), off), ds));
    }
#pragma unroll
    for (int c = 0; c < 4; c++) store_chunk(tile, m, 4 * h + c, make_uint4(o[4 * c], o[4 * c + 1], o[4 * c + 2], o[4 * c + 3]));
  }
};

// IQ3_S: w = d * (1 + 2 s) * grid[index][i] * sign. A half is one sub-block of 32: 8 bytes of qs, a byte of qh, 4 of
// signs, a nibble of scale. The codebook is in shared memory.
template <>
struct Decoder<QT_IQ3_S> {
  static constexpr uint32_t kStageBytes = 16;  // bytes of a row's main quants run a 64-value stage reads
  struct Hdr {};
  __device__ static __forceinline__ Hdr fetch_hdr(const uint8_t *, uint64_t, uint32_t, uint32_t, uint32_t) { return Hdr{}; }
  struct Raw {
    uint2 qs;
    uint32_t sg, qh, sc;
    __half d;
  };
  __device__ static __forceinline__ const uint8_t *quants_at(const uint8_t *s, uint64_t, uint32_t K, uint32_t r, uint32_t k0, uint32_t h) {
    return s + 64 * ((uint64_t)r * (K / 256) + k0 / 256) + 8 * ((k0 % 256) / 32 + h);
  }
  __device__ static __forceinline__ Raw fetch(const uint8_t *s, uint64_t nblk, uint32_t K, uint32_t r, uint32_t k0, uint32_t h) {
    const uint32_t sb = (k0 % 256) / 32 + h;  // the sub-block within its block
    const uint64_t blk = (uint64_t)r * (K / 256) + k0 / 256;
    Raw x;
    x.qs = __ldg((const uint2 *)(s + 64 * blk + 8 * sb));
    x.sg = __ldg((const uint32_t *)(s + 64 * nblk + 32 * blk + 4 * sb));
    x.qh = __ldg(s + 96 * nblk + 8 * blk + sb);
    x.sc = (__ldg(s + 104 * nblk + 4 * blk + sb / 2) >> (4 * (sb & 1))) & 0xF;
    x.d = __ldg((const __half *)(s + 108 * nblk) + blk);
    return x;
  }
  __device__ static __forceinline__ void store(const Hdr &, const Raw &x, uint8_t *tile, uint32_t m, uint32_t h, uint32_t, const uint32_t *grid) {
    const __half2 ls = small_h2(2 * x.sc + 1), d2 = __half2half2(x.d), off = as_h2(0x64006400u);
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
    for (int c = 0; c < 4; c++) store_chunk(tile, m, 4 * h + c, make_uint4(o[4 * c], o[4 * c + 1], o[4 * c + 2], o[4 * c + 3]));
  }
};

// Four codebook bytes (a word of values below 128) times sc as f16 with the nibble's signs, into o[0], o[1].
__device__ __forceinline__ void grid_word_to_f16(uint32_t g, uint32_t nib, __half2 sc, uint32_t *o) {
  const __half2 off = as_h2(0x64006400u);
  // The sign bit of each f16: values 0, 1 from the nibble's bits 0, 1; 2, 3 from bits 2, 3.
  const uint32_t s01 = ((nib & 1u) << 15) | ((nib & 2u) << 30), s23 = ((nib & 4u) << 13) | ((nib & 8u) << 28);
  o[0] = as_u32(__hmul2(__hsub2(as_h2(bias_h2(g, 0x4140)), off), sc)) ^ s01;
  o[1] = as_u32(__hmul2(__hsub2(as_h2(bias_h2(g, 0x4342)), off), sc)) ^ s23;
}

// IQ3_XXS: w = d * (0.5 + s) / 2 * grid[index][i] * sign. A half is one sub-block of 32: 8 bytes of indices and its
// word of four 7-bit sign indices and the scale. The codebook is in shared memory.
template <>
struct Decoder<QT_IQ3_XXS> {
  static constexpr uint32_t kStageBytes = 16;  // bytes of a row's main quants run a 64-value stage reads
  struct Hdr {};
  __device__ static __forceinline__ Hdr fetch_hdr(const uint8_t *, uint64_t, uint32_t, uint32_t, uint32_t) { return Hdr{}; }
  struct Raw {
    uint2 qs;
    uint32_t w32;
    __half d;
  };
  __device__ static __forceinline__ const uint8_t *quants_at(const uint8_t *s, uint64_t, uint32_t K, uint32_t r, uint32_t k0, uint32_t h) {
    return s + 64 * ((uint64_t)r * (K / 256) + k0 / 256) + 8 * ((k0 % 256) / 32 + h);
  }
  __device__ static __forceinline__ Raw fetch(const uint8_t *s, uint64_t nblk, uint32_t K, uint32_t r, uint32_t k0, uint32_t h) {
    const uint32_t sb = (k0 % 256) / 32 + h;  // the sub-block within its block
    const uint64_t blk = (uint64_t)r * (K / 256) + k0 / 256;
    Raw x;
    x.qs = __ldg((const uint2 *)(s + 64 * blk + 8 * sb));
    x.w32 = __ldg((const uint32_t *)(s + 64 * nblk + 32 * blk + 4 * sb));
    x.d = __ldg((const __half *)(s + 96 * nblk) + blk);
    return x;
  }
  __device__ static __forceinline__ void store(const Hdr &, const Raw &x, uint8_t *tile, uint32_t m, uint32_t h, uint32_t, const uint32_t *grid) {
    // d * (2 s + 1) / 4, rounded to f16 once.
    const __half2 sc = __float2half2_rn(__half2float(x.d) * (float)(2 * (x.w32 >> 28) + 1) * 0.25f);
    uint32_t o[16];
#pragma unroll
    for (int k = 0; k < 8; k++) {
      const uint32_t word = k < 4 ? x.qs.x : x.qs.y;
      const uint32_t k7 = (x.w32 >> (7 * (k >> 1))) & 127u, sbyte = k7 | ((__popc(k7) & 1u) << 7);
      grid_word_to_f16(grid[(word >> (8 * (k & 3))) & 0xFF], (sbyte >> (4 * (k & 1))) & 0xF, sc, o + 2 * k);
    }
#pragma unroll
    for (int c = 0; c < 4; c++) store_chunk(tile, m, 4 * h + c, make_uint4(o[4 * c], o[4 * c + 1], o[4 * c + 2], o[4 * c + 3]));
  }
};

// IQ2_S: w = d * (0.5 + s) / 4 * grid[index][i] * sign. A half is one sub-block of 32: four groups of 8 values, each a
// 10-bit index (a byte of qs, two bits of the sub-block's qh byte) and a byte of signs; a scale nibble per two groups.
template <>
struct Decoder<QT_IQ2_S> {
  static constexpr uint32_t kStageBytes = 8;  // bytes of a row's main quants run a 64-value stage reads
  struct Hdr {};
  __device__ static __forceinline__ Hdr fetch_hdr(const uint8_t *, uint64_t, uint32_t, uint32_t, uint32_t) { return Hdr{}; }
  struct Raw {
    uint32_t qs, sg, qh, sc;
    __half d;
  };
  __device__ static __forceinline__ const uint8_t *quants_at(const uint8_t *s, uint64_t, uint32_t K, uint32_t r, uint32_t k0, uint32_t h) {
    return s + 32 * ((uint64_t)r * (K / 256) + k0 / 256) + 4 * ((k0 % 256) / 32 + h);
  }
  __device__ static __forceinline__ Raw fetch(const uint8_t *s, uint64_t nblk, uint32_t K, uint32_t r, uint32_t k0, uint32_t h) {
    const uint32_t sb = (k0 % 256) / 32 + h;
    const uint64_t blk = (uint64_t)r * (K / 256) + k0 / 256;
    Raw x;
    x.qs = __ldg((const uint32_t *)(s + 32 * blk + 4 * sb));
    x.sg = __ldg((const uint32_t *)(s + 32 * nblk + 32 * blk + 4 * sb));
    x.qh = __ldg(s + 64 * nblk + 8 * blk + sb);
    x.sc = __ldg(s + 72 * nblk + 8 * blk + sb);
    x.d = __ldg((const __half *)(s + 80 * nblk) + blk);
    return x;
  }
  __device__ static __forceinline__ void store(const Hdr &, const Raw &x, uint8_t *tile, uint32_t m, uint32_t h, uint32_t, const uint32_t *grid) {
    const float d8 = __half2float(x.d) * 0.125f;  // d * (2 s + 1) / 8
    const __half2 sc_lo = __float2half2_rn(d8 * (float)(2 * (x.sc & 0xF) + 1)), sc_hi = __float2half2_rn(d8 * (float)(2 * (x.sc >> 4) + 1));
    const uint2 *grid2 = (const uint2 *)grid;
#pragma unroll
    for (int g = 0; g < 4; g++) {
      const uint2 e = grid2[((x.qs >> (8 * g)) & 0xFF) | (((x.qh >> (2 * g)) & 3u) << 8)];
      const uint32_t sb = (x.sg >> (8 * g)) & 0xFF;
      uint32_t o[4];
      grid_word_to_f16(e.x, sb & 0xF, g < 2 ? sc_lo : sc_hi, o), grid_word_to_f16(e.y, sb >> 4, g < 2 ? sc_lo : sc_hi, o + 2);
      store_chunk(tile, m, 4 * h + g, make_uint4(o[0], o[1], o[2], o[3]));
    }
  }
};

// Sixteen table values (four words of signed bytes) times d2 as f16, into o[0 .. 7].
__device__ __forceinline__ void int8x16_to_f16(const uint32_t (&w)[4], __half2 d2, uint32_t *o) {
  const __half2 off = as_h2(0x64806480u);  // 1152 = 1024 + 128
#pragma unroll
  for (int j = 0; j < 4; j++) {
    const uint32_t u = w[j] ^ 0x80808080u;  // int8 + 128
    o[2 * j] = as_u32(__hmul2(__hsub2(as_h2(bias_h2(u, 0x4140)), off), d2));
    o[2 * j + 1] = as_u32(__hmul2(__hsub2(as_h2(bias_h2(u, 0x4342)), off), d2));
  }
}
// A block or sub-block of 32 four-bit codes (16 bytes: values 0 .. 15 in the low nibbles, 16 .. 31 in the high ones)
// through the table, times d2, into chunks 4 h .. 4 h + 3 of the row.
__device__ __forceinline__ void iq4_store32(const uint4 &q, __half2 d2, uint8_t *tile, uint32_t m, uint32_t h) {
  uint32_t lo[4], hi[4], o[16];
  iq4_lookup8(q.x, lo[0], hi[0]), iq4_lookup8(q.y, lo[1], hi[1]), iq4_lookup8(q.z, lo[2], hi[2]), iq4_lookup8(q.w, lo[3], hi[3]);
  int8x16_to_f16(lo, d2, o), int8x16_to_f16(hi, d2, o + 8);
#pragma unroll
  for (int c = 0; c < 4; c++) store_chunk(tile, m, 4 * h + c, make_uint4(o[4 * c], o[4 * c + 1], o[4 * c + 2], o[4 * c + 3]));
}

// Q2_0: w = (q - 1) * d. A stage is one block of 64; a half is 8 of its 16 bytes.
template <>
struct Decoder<QT_Q2_0> {
  static constexpr uint32_t kStageBytes = 16;  // bytes of a row's main quants run a 64-value stage reads
  struct Hdr {};
  __device__ static __forceinline__ Hdr fetch_hdr(const uint8_t *, uint64_t, uint32_t, uint32_t, uint32_t) { return Hdr{}; }
  struct Raw {
    uint2 q;
    __half d;
  };
  __device__ static __forceinline__ const uint8_t *quants_at(const uint8_t *s, uint64_t, uint32_t K, uint32_t r, uint32_t k0, uint32_t h) {
    return s + (uint64_t)r * (K / 4) + k0 / 4 + 8 * h;
  }
  __device__ static __forceinline__ Raw fetch(const uint8_t *s, uint64_t nblk, uint32_t K, uint32_t r, uint32_t k0, uint32_t h) {
    Raw x;
    x.q = __ldg((const uint2 *)quants_at(s, nblk, K, r, k0, h));
    x.d = __ldg((const __half *)(s + 16 * nblk) + (uint64_t)r * (K / 64) + k0 / 64);
    return x;
  }
  __device__ static __forceinline__ void store(const Hdr &, const Raw &x, uint8_t *tile, uint32_t m, uint32_t h, uint32_t, const uint32_t *) {
    uint32_t w[8], o[16];
#pragma unroll
    for (int i = 0; i < 8; i++) w[i] = q2_bytes(((i < 4 ? x.q.x : x.q.y) >> (8 * (i & 3))) & 0xFF);
    const __half2 d2 = __half2half2(x.d);
    int8x16_to_f16(*(const uint32_t(*)[4])&w[0], d2, o), int8x16_to_f16(*(const uint32_t(*)[4])&w[4], d2, o + 8);
#pragma unroll
    for (int c = 0; c < 4; c++) store_chunk(tile, m, 4 * h + c, make_uint4(o[4 * c], o[4 * c + 1], o[4 * c + 2], o[4 * c + 3]));
  }
};

// IQ4_NL: w = d * table[q]. A half is one block of 32.
template <>
struct Decoder<QT_IQ4_NL> {
  static constexpr uint32_t kStageBytes = 32;  // bytes of a row's main quants run a 64-value stage reads
  struct Hdr {};
  __device__ static __forceinline__ Hdr fetch_hdr(const uint8_t *, uint64_t, uint32_t, uint32_t, uint32_t) { return Hdr{}; }
  struct Raw {
    uint4 q;
    __half d;
  };
  __device__ static __forceinline__ const uint8_t *quants_at(const uint8_t *s, uint64_t, uint32_t K, uint32_t r, uint32_t k0, uint32_t h) {
    return s + (uint64_t)r * (K / 2) + k0 / 2 + 16 * h;
  }
  __device__ static __forceinline__ Raw fetch(const uint8_t *s, uint64_t nblk, uint32_t K, uint32_t r, uint32_t k0, uint32_t h) {
    Raw x;
    x.q = ldg16(quants_at(s, nblk, K, r, k0, h));
    x.d = __ldg((const __half *)(s + 16 * nblk) + (uint64_t)r * (K / 32) + k0 / 32 + h);
    return x;
  }
  __device__ static __forceinline__ void store(const Hdr &, const Raw &x, uint8_t *tile, uint32_t m, uint32_t h, uint32_t, const uint32_t *) {
    iq4_store32(x.q, __half2half2(x.d), tile, m, h);
  }
};

// IQ4_XS: w = d * (ls - 32) * table[q]. A half is one sub-block of 32 with its 6-bit ls.
template <>
struct Decoder<QT_IQ4_XS> {
  static constexpr uint32_t kStageBytes = 32;  // bytes of a row's main quants run a 64-value stage reads
  struct Hdr {};
  __device__ static __forceinline__ Hdr fetch_hdr(const uint8_t *, uint64_t, uint32_t, uint32_t, uint32_t) { return Hdr{}; }
  struct Raw {
    uint4 q;
    uint32_t ls;
    __half d;
  };
  __device__ static __forceinline__ const uint8_t *quants_at(const uint8_t *s, uint64_t, uint32_t K, uint32_t r, uint32_t k0, uint32_t h) {
    return s + (uint64_t)r * (K / 2) + k0 / 2 + 16 * h;
  }
  __device__ static __forceinline__ Raw fetch(const uint8_t *s, uint64_t nblk, uint32_t K, uint32_t r, uint32_t k0, uint32_t h) {
    const uint32_t ib = (k0 % 256) / 32 + h;  // the sub-block within its block
    const uint64_t blk = (uint64_t)r * (K / 256) + k0 / 256;
    Raw x;
    x.q = ldg16(quants_at(s, nblk, K, r, k0, h));
    const uint32_t sl = __ldg((const uint32_t *)(s + 128 * nblk) + blk), sh = __ldg((const uint16_t *)(s + 132 * nblk) + blk);
    x.ls = ((sl >> (4 * ib)) & 0xF) | (((sh >> (2 * ib)) & 3) << 4);
    x.d = __ldg((const __half *)(s + 134 * nblk) + blk);
    return x;
  }
  __device__ static __forceinline__ void store(const Hdr &, const Raw &x, uint8_t *tile, uint32_t m, uint32_t h, uint32_t, const uint32_t *) {
    // d * (ls - 32) rounded to f16 once; ls - 32 is in -32 .. 31, exact in f16.
    iq4_store32(x.q, __float2half2_rn(__half2float(x.d) * (float)((int)x.ls - 32)), tile, m, h);
  }
};

}  // namespace tc


// Whether a type's quants reach the decode warps through a ring in shared memory filled by bulk-tensor copies, rather
// than by the warps' own global loads (whose one-row-per-lane pattern costs the load pipe 32 wavefronts an
// instruction). Q4_K, the benchmark's type: its quants are one run of K / 2 bytes a row, which a 3-D map (bytes of the
// row, rows, expert slots) covers.
__host__ __device__ constexpr bool quants_by_copy(uint32_t qt) { return qt == QT_Q4_K; }

// Shared memory of a CTA: the stages (NMAT weight tiles of 16 KB and a row tile of 32 KB each), then (for types whose
// quants come by copy) a ring of two quant slots, then the barriers, then a codebook type's codebook.
// A quant slot holds, for every weight row of the item, the quants of one stage per decode group: 32 bytes a stage for
// Q4_K, so 64 bytes a row with two groups (64-byte swizzle) and 128 with four (128-byte swizzle).
template <int QT, int NMAT, bool PAIR = false>
struct TileSmem {
  // A CTA of a pair holds half the rows' tile, which leaves room for more stages.
  static constexpr uint32_t kStages = PAIR ? (NMAT == 2 ? 4 : 6) : (NMAT == 2 ? 3 : 4);
  static constexpr uint32_t kXRows = PAIR ? kTileN / 2 : kTileN;
  static constexpr uint32_t kWBytes = kTileM * kTileK * 2, kXBytes = kXRows * kTileK * 2;
  static constexpr uint32_t kStageBytes = NMAT * kWBytes + kXBytes;
  static constexpr uint32_t kGroups = kTileDecoders / (NMAT * kTileM);                // decode groups: 2 or 4
  static constexpr uint32_t kQRowBytes = kGroups * 32;                                // a row's bytes in a quant slot
  static constexpr uint32_t kQMatBytes = kTileM * kQRowBytes, kQSlotBytes = NMAT * kQMatBytes, kQSlots = 2;
  static constexpr uint32_t kQuants = kStages * kStageBytes;
  static constexpr uint32_t kBarriers = kQuants + (quants_by_copy(QT) ? kQSlots * kQSlotBytes : 0);
  // full[kStages], empty[kStages], accumulators full[2], empty[2], empty after a two-buffer item, quant slots full[2],
  // empty[2]; tmem address; abort
  static constexpr uint32_t kGrid = kBarriers + 256;                                  // the codebook: 1, 2 or 8 KB
  static constexpr uint32_t kBytes = kGrid + 4 * grid_words(QT) + 1024;               // and room to align the base to 1024
  static_assert(kBytes <= 227 * 1024, "a CTA's shared memory");
};

// SwiGLU with the fast exponential and division: the tensor-core path's results already differ from the CPU path's
// in the last bits of f16 products, so full-precision expf buys nothing here.
__device__ __forceinline__ float swiglu_fast(float g, float u, float limit) {
  if (limit > 0.0f) {
    g = fminf(g, limit);
    u = fminf(fmaxf(u, -limit), limit);
  }
  return __fdividef(g, 1.0f + __expf(-g)) * u;
}


// The tile a work item belongs to.
struct ItemTile {
  uint32_t slot, start, count;
};
__device__ __forceinline__ ItemTile item_tile(const ExpertTilesArgs &a, uint32_t ti) {
  if (a.tiles) {
    const BigTile t = a.tiles[ti];
    return ItemTile{t.slot, t.start, t.count};
  }
  const uint32_t start = ti * kTileN;
  return ItemTile{0, start, min(kTileN, a.dense_rows - start)};
}

// NMAT 2: out = swiglu(gate x, up x); NMAT 1: out = down h. Persistent: the grid is one CTA per SM (fewer when there is
// less work), single or in pairs (PAIR, below); a unit (a CTA or a pair) takes the work items dealt to it round by
// round; item i is weight-row tile (or pair of tiles) i % RTU of big tile i / RTU, so neighbouring units share a tile's
// activations in L2. Five roles: 16 decode warps (quants to f16 weights in shared memory), 4 epilogue warps
// (accumulators to the result), a warp whose first lane issues the bulk-tensor copies of the rows' activations (the
// whole warp when the rows are gathered by index), the warp that owns tensor memory and whose first lane issues the
// MMAs, and a warp whose first lane issues the copies of the quants for types that take them through the ring. A warp
// arrives on a barrier once, by one lane.
//
// Tensor memory is two buffers of 256 columns. An item of at most 128 rows (any item, for NMAT 1) takes one buffer,
// alternately, so the epilogue warps drain item i while the MMAs of item i + 1 run and the decode warps never stop. A
// gate/up item of more than 128 rows needs both buffers (gate in one, up in the other): the MMAs of the next item
// wait for its epilogue, and to keep that short the decode warps join the epilogue warps for it.
// Dynamic shared memory TileSmem::kBytes.
template <int QT, int NMAT, bool PAIR>
__global__ void __launch_bounds__(kTileThreads, 1) k_expert_tiles(const __grid_constant__ ExpertTilesArgs a,
                                                                  const __grid_constant__ CUtensorMap act_map,
                                                                  const uint32_t *__restrict__ grid_global) {
  using namespace tc;
  using SM = TileSmem<QT, NMAT, PAIR>;
  using Dec = Decoder<QT>;
  using Raw = typename Dec::Raw;
  constexpr uint32_t S = SM::kStages, kCols = 512;
  constexpr uint32_t kDW = kTileDecoders / 32, kEW = kTileEpilogue / 32, kCopyWarp = kDW + kEW, kMmaWarp = kCopyWarp + 1, kQuantWarp = kMmaWarp + 1;
  // A decode thread takes a whole row of a stage, 64 values as two halves of 32, so that what a stage costs a thread
  // beside the arithmetic (the barrier round trip, the addresses, the block's scales) is paid once per 64 values. A
  // stage's NMAT * 128 rows are one group of threads; the 512 decode threads form 2 groups (two matrices) or 4 (one),
  // and group g takes stages g, g + groups, ...
  constexpr uint32_t kGroupThreads = NMAT * kTileM, kDecGroups = kTileDecoders / kGroupThreads;
  extern __shared__ uint8_t smem_raw[];
  uint8_t *smem = (uint8_t *)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);

  const uint32_t K = a.K, KT = K / kTileK, RT = a.R / kTileM;
  const uint32_t ntiles = a.tiles ? *a.ntiles : (a.dense_rows + kTileN - 1) / kTileN;
  // PAIR: the CTAs come in clusters of two, on the two SMs of a TPC. A pair is one unit of work: its item is 256 weight
  // rows (128 decoded by each CTA) times the tile's rows, of which each CTA brings half into its own shared memory;
  // the first CTA's MMA thread issues one tcgen05.mma.cta_group::2 for both, which reads both halves and writes each
  // CTA's 128 weight rows of the product into that CTA's tensor memory. What a CTA's shared memory carries per flop
  // is the weights as before but only half the rows, and shared-memory bandwidth is what bounds the single-CTA form.
  const uint32_t rank = PAIR ? cluster_ctarank() : 0;
  const uint32_t unit = PAIR ? blockIdx.x / 2 : blockIdx.x, nunits = PAIR ? gridDim.x / 2 : gridDim.x;
  const uint32_t RTU = PAIR ? RT / 2 : RT;  // a big tile's items
  const uint32_t nitems = ntiles * RTU;
  if (unit >= nitems) return;  // both CTAs of a pair alike
  const uint32_t tid = threadIdx.x, warp = tid / 32, lane = tid % 32;
  uint64_t *bars = (uint64_t *)(smem + SM::kBarriers);
  const uint32_t bar0 = smem_u32(bars);
  auto full_bar = [&](uint32_t s) { return bar0 + 8 * s; };
  auto empty_bar = [&](uint32_t s) { return bar0 + 8 * (S + s); };
  auto acc_full = [&](uint32_t b) { return bar0 + 8 * (2 * S + b); };
  auto acc_empty = [&](uint32_t b) { return bar0 + 8 * (2 * S + 2 + b); };
  const uint32_t acc_empty_wide = bar0 + 8 * (2 * S + 4);
  auto q_full = [&](uint32_t b) { return bar0 + 8 * (2 * S + 5 + b); };
  auto q_empty = [&](uint32_t b) { return bar0 + 8 * (2 * S + 7 + b); };
  uint32_t *tmem_slot = (uint32_t *)(bars + 2 * S + 9);
  volatile uint32_t *abort = tmem_slot + 1;
  uint32_t *grid = (uint32_t *)(smem + SM::kGrid);

  // A stage is full when every decode warp has stored its weights (one arrival a warp) and the rows' copies have landed
  // (the copy thread's arrival states their bytes; the copy unit counts them off). An accumulator buffer is empty again
  // when the epilogue warps have read it; after an item that took both buffers, also when the decode warps have.
  if (tid == 0) {
    // In a pair the first CTA's full, accumulator-empty barriers take both CTAs' arrivals.
    constexpr uint32_t kCtas = PAIR ? 2 : 1;
    for (uint32_t s = 0; s < S; s++) mbar_init(full_bar(s), kCtas * (kDW / kDecGroups + 1)), mbar_init(empty_bar(s), 1);
    for (uint32_t b = 0; b < 2; b++) mbar_init(acc_full(b), 1), mbar_init(acc_empty(b), kCtas * kEW);
    mbar_init(acc_empty_wide, kCtas * kDW);
    for (uint32_t b = 0; b < 2; b++) mbar_init(q_full(b), 1), mbar_init(q_empty(b), kDW);
    *abort = 0;
    fence_barrier_init();
  }
  if constexpr (grid_words(QT) > 0)
    for (uint32_t i = tid; i < grid_words(QT); i += blockDim.x) grid[i] = grid_global[grid_offset(QT) + i];
  if (warp == kMmaWarp) {
    if constexpr (PAIR)
      tmem_alloc_pair(smem_u32(tmem_slot), kCols);  // the same warp of both CTAs, the same place for the address
    else
      tmem_alloc(smem_u32(tmem_slot), kCols);
  }
  tc_fence_before();
  __syncthreads();
  if constexpr (PAIR) cluster_sync();  // the other CTA's barriers exist before anything arrives on them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  bool ok = true;
  // The first CTA's barriers, as the pair's other CTA names them (for the first CTA itself: its own).
  const uint32_t bar0_lead = PAIR ? map_to_cta(bar0, 0) : bar0;
  auto full_lead = [&](uint32_t s) { return bar0_lead + 8 * s; };
  auto acc_empty_lead = [&](uint32_t b) { return bar0_lead + 8 * (2 * S + 2 + b); };
  const uint32_t acc_empty_wide_lead = bar0_lead + 8 * (2 * S + 4);
  // Arrivals that in a pair go to the first CTA's barrier.
  auto arrive_lead = [&](uint32_t lead_bar, uint32_t own_bar) {
    if constexpr (PAIR)
      mbar_arrive_cluster(lead_bar);
    else
      mbar_arrive(own_bar);
  };
  // The weight rows of an item that this CTA decodes and drains.
  auto item_rows0 = [&](uint32_t item) { return ((item % RTU) * (PAIR ? 2u : 1u) + rank) * kTileM; };

  // CTA b's item of round r: the items come expert by expert for the experts with full tiles, then the short tiles of
  // the others by falling row count, and the rounds deal them boustrophedon (b, then G - 1 - b, ...), so that every CTA
  // gets a like share of long and short items. kNoItem past the end; a CTA's last round may have no item for it while others still have one.
  constexpr uint32_t kNoItem = 0xFFFFFFFFu;
  auto item_at = [&](uint32_t rnd) {
    const uint32_t base = rnd * nunits;
    const uint32_t i = base + ((rnd & 1) ? nunits - 1 - unit : unit);
    return i < nitems ? i : kNoItem;
  };

  // Every role walks the same items and keeps the same books: how often each buffer has been used (the parity of its
  // barriers' phases), which buffer the next one-buffer item takes, and how many two-buffer items there have been.
  uint32_t use0 = 0, use1 = 0, next_buf = 0, wides = 0;  // two scalars, not an array: they stay in registers
  auto use_of = [&](uint32_t b) { return b ? use1 : use0; };
  auto use_inc = [&](uint32_t b) { use0 += b == 0, use1 += b == 1; };
  auto is_wide = [&](uint32_t count) { return NMAT == 2 && count > kTileN / 2; };

  // Columns q (this warp's quarter of the weight rows: TMEM lanes 32 q ..) of chunks slot, slot + nslots, ... of W rows
  // each, from the accumulators at column colg (and colu, the up product) to the result. A lane holds one weight row's
  // values for the chunk's W rows; for each row the warp's 32 lanes store 32 consecutive values. The address of a
  // chunk is worked out once and stepped by the row stride: what the loop costs per value is a conversion and a store.
  // The loads of a warp's next chunk are in flight while it converts and stores the one before (two sets of
  // registers): what a chunk costs is then its instructions, not tensor memory's latency, which alone had the down
  // product's four epilogue warps take longer over an item than its MMAs do.
  auto drain = [&](const ItemTile &t, uint32_t r0, uint32_t colg, uint32_t colu, uint32_t slot, uint32_t nslots) {
    constexpr int W = NMAT == 2 ? 8 : 16;
    const uint32_t q = warp % 4, r = r0 + 32 * q + lane, nch = ((t.count + 15) & ~15u) / W;
    const uint32_t lanes = tmem_base + ((32 * q) << 16);
    auto load = [&](uint32_t c, uint32_t *g, uint32_t *u) {
      if constexpr (NMAT == 2)
        tmem_ld8(lanes + colg + W * c, g), tmem_ld8(lanes + colu + W * c, u);
      else
        tmem_ld16(lanes + colg + W * c, g);
    };
    auto wait = [&](uint32_t *g, uint32_t *u) {
      if constexpr (NMAT == 2)
        tmem_ld_wait8(g), tmem_ld_wait8(u);
      else
        tmem_ld_wait16(g);
    };
    auto store = [&](uint32_t c, const uint32_t *g, const uint32_t *u) {
      if (W * c >= t.count) return;           // a chunk of rows past the tile's (the rows are rounded up to 16)
      const uint32_t left = t.count - W * c;  // rows of the chunk that exist
      float v[W];
#pragma unroll
      for (int j = 0; j < W; j++) {
        v[j] = __uint_as_float(g[j]);
        if constexpr (NMAT == 2) v[j] = swiglu_fast(v[j], __uint_as_float(u[j]), a.limit);
      }
      const uint64_t at = (uint64_t)(t.start + W * c) * a.out_stride + r;
      if (a.out_f16) {
        __half *p = (__half *)a.out + at;
        if (left >= (uint32_t)W) {
#pragma unroll
          for (int j = 0; j < W; j++) p[(uint64_t)j * a.out_stride] = __float2half_rn(v[j]);
        } else {
#pragma unroll
          for (int j = 0; j < W; j++)
            if ((uint32_t)j < left) p[(uint64_t)j * a.out_stride] = __float2half_rn(v[j]);
        }
      } else {
        float *p = (float *)a.out + at;
        if (left >= (uint32_t)W) {
#pragma unroll
          for (int j = 0; j < W; j++) p[(uint64_t)j * a.out_stride] = v[j];
        } else {
#pragma unroll
          for (int j = 0; j < W; j++)
            if ((uint32_t)j < left) p[(uint64_t)j * a.out_stride] = v[j];
        }
      }
    };
    uint32_t gA[W], gB[W], uA[NMAT == 2 ? W : 1], uB[NMAT == 2 ? W : 1];
    uint32_t c = slot;
    if (c >= nch) return;
    load(c, gA, uA);
    for (;;) {
      wait(gA, uA);
      uint32_t cn = c + nslots;
      if (cn < nch) load(cn, gB, uB);
      store(c, gA, uA);
      if (cn >= nch) break;
      c = cn, cn = c + nslots;
      wait(gB, uB);
      if (cn < nch) load(cn, gA, uA);
      store(c, gB, uB);
      if (cn >= nch) break;
      c = cn;
    }
  };

  if (warp < kDW) {
    // Decode warps. 8 consecutive threads take the 8 rows of a core matrix, so a quarter-warp's 16-byte stores fill 128
    // contiguous bytes.
    const uint64_t nblk = (uint64_t)a.R * (K / block_values(QT));
    const uint32_t first = tid / kGroupThreads, mat = (tid % kGroupThreads) / kTileM, m = tid % kTileM;
    uint32_t li = 0;
    // For types whose quants come by copy, the one thing a decode thread still loads itself is a block's header, and it
    // asks for it a block ahead (across items too), so that no stage begins by waiting for it: hdr_ahead holds the
    // header of the next block the thread will decode.
    typename Dec::Hdr hdr_ahead;
    if constexpr (quants_by_copy(QT)) {
      const uint32_t i0 = item_at(0);
      if (i0 != kNoItem && first < KT) {
        const ItemTile t0 = item_tile(a, i0 / RTU);
        hdr_ahead = Dec::fetch_hdr((mat == 0 ? a.w0 : a.w1) + (uint64_t)t0.slot * a.slice_bytes, nblk, K, item_rows0(i0) + m,
                                   (first * kTileK) & ~255u);
      }
    }
    for (uint32_t rnd = 0, item; (item = item_at(rnd)) != kNoItem && ok; rnd++, li++) {
      const ItemTile t = item_tile(a, item / RTU);
      const uint32_t r0 = item_rows0(item);
      const uint8_t *wm = (mat == 0 ? a.w0 : a.w1) + (uint64_t)t.slot * a.slice_bytes;
      // The next item's weights and rows, known early: its first header is asked for at this item's last stage.
      const uint32_t item_after = quants_by_copy(QT) ? item_at(rnd + 1) : kNoItem;
      ItemTile t_after{0, 0, 0};
      if (item_after != kNoItem) t_after = item_tile(a, item_after / RTU);
      // Quants come from HBM the first time an expert is touched; a request for the L2 goes out kAhead stages before
      // the load into registers, which itself goes a stage of this thread's before the decode.
      constexpr uint32_t kLineStages = 128 / Dec::kStageBytes;
      constexpr uint32_t kAhead = kLineStages > 6 ? kLineStages : 6 / kLineStages * kLineStages;  // a whole number of lines, about 6 stages
      Raw raw[2][2];  // [buffer][half]
      // The block's scales travel with the stage's quants: loaded when a stage is the thread's first in its block, kept
      // for its later stages there.
      typename Dec::Hdr hdr[2], hdr_last;
      uint32_t blk_fetched = 0xFFFFFFFFu;
      auto fetch = [&](uint32_t b, uint32_t it) {
        const uint32_t k0 = it * kTileK;
        if constexpr (quants_by_copy(QT)) {
          // The header asked for a block ago is this block's; the one after it is asked for now.
          if (it == first || k0 / 256 != blk_fetched) hdr_last = hdr_ahead, blk_fetched = k0 / 256;
          const uint32_t it2 = it + kDecGroups;
          if (it2 < KT) {
            if (it2 * kTileK / 256 != blk_fetched) hdr_ahead = Dec::fetch_hdr(wm, nblk, K, r0 + m, (it2 * kTileK) & ~255u);
          } else if (item_after != kNoItem) {
            hdr_ahead = Dec::fetch_hdr((mat == 0 ? a.w0 : a.w1) + (uint64_t)t_after.slot * a.slice_bytes, nblk, K,
                                       item_rows0(item_after) + m, (first * kTileK) & ~255u);
          }
        } else {
          if (k0 / 256 != blk_fetched) hdr_last = Dec::fetch_hdr(wm, nblk, K, r0 + m, k0 & ~255u), blk_fetched = k0 / 256;
        }
        hdr[b] = hdr_last;
        if constexpr (quants_by_copy(QT)) {
          // The stage's 32 bytes of this row from the quant ring: slot qn holds one stage per group, this group's at
          // bytes 32 * first of the row, its 16-byte pieces swizzled by the row as the copy laid them.
          const uint32_t qn = li * (KT / kDecGroups) + it / kDecGroups, qb = qn % SM::kQSlots;
          if (!mbar_wait(q_full(qb), (qn / SM::kQSlots) & 1, abort, a.error)) {
            ok = false;
            return;
          }
          const uint8_t *row = smem + SM::kQuants + qb * SM::kQSlotBytes + mat * SM::kQMatBytes + m * SM::kQRowBytes;
          const uint32_t sw = SM::kQRowBytes == 64 ? (m >> 1) & 3 : m & 7;
          raw[b][0].q = *(const uint4 *)(row + 16 * ((2 * first) ^ sw));
          raw[b][1].q = *(const uint4 *)(row + 16 * ((2 * first + 1) ^ sw));
          // These reads are the generic proxy's and the copy that refills the slot is the async proxy's: without the
          // fence the copy was seen to overtake them (a few 128-byte lines of a slot read as the next stage's quants,
          // run to run different). The fence orders the reads before whatever the arrival below lets loose.
          fence_async_smem();
          __syncwarp();
          if (lane == 0) mbar_arrive(q_empty(qb));
        } else {
          raw[b][0] = Dec::fetch(wm, nblk, K, r0 + m, k0, 0);
          raw[b][1] = Dec::fetch(wm, nblk, K, r0 + m, k0, 1);
          // One request a 128-byte line, which holds kLineStages stages of the row.
          if (it % kLineStages == 0 && k0 + kAhead * kTileK < K) prefetch_l2(Dec::quants_at(wm, nblk, K, r0 + m, k0 + kAhead * kTileK, 0));
        }
      };
      auto stage_step = [&](uint32_t b, uint32_t it) {
        const uint32_t g = li * KT + it, s = g % S, use_s = g / S, k0 = it * kTileK;
        if (use_s > 0) ok = mbar_wait(empty_bar(s), (use_s - 1) & 1, abort, a.error);
        if (!ok) return;
        tc_fence_after();
        uint8_t *tile = smem + s * SM::kStageBytes + mat * SM::kWBytes;
        Dec::store(hdr[b], raw[b][0], tile, m, 0, k0, grid);
        Dec::store(hdr[b], raw[b][1], tile, m, 1, k0, grid);
        fence_async_smem();
        __syncwarp();
        if (lane == 0) arrive_lead(full_lead(s), full_bar(s));
      };
      // The first lines of a row's quants are asked for an item ahead (below), so that an item does not begin by
      // waiting for HBM; the CTA's first item asks for its own.
      auto ask_ahead = [&](const uint8_t *w, uint32_t row) {
        for (uint32_t p = 0; p < kAhead && p < KT; p += kLineStages) prefetch_l2(Dec::quants_at(w, nblk, K, row, p * kTileK, 0));
      };
      if (!quants_by_copy(QT) && first == 0 && li == 0) ask_ahead(wm, r0 + m);
      const uint32_t item_next = quants_by_copy(QT) ? kNoItem : item_at(rnd + 1);
      // This thread's stages: first, first + kDecGroups, ...; the quants of one are loaded while the one before decodes.
      if constexpr (quants_by_copy(QT)) {
        // The quants wait in shared memory: nothing to load ahead; a stage is read and decoded in one go.
        for (uint32_t it = first; it < KT && ok; it += kDecGroups) {
          fetch(0, it);
          if (ok) stage_step(0, it);
        }
      } else {
      if (first < KT) fetch(0, first);
      for (uint32_t it = first; it < KT && ok; it += 2 * kDecGroups) {
        if (it + kDecGroups < KT) fetch(1, it + kDecGroups);
        stage_step(0, it);
        if (it == 0 && item_next != kNoItem) {  // group 0, after its first stage: the next item's first lines
          const ItemTile tn = item_tile(a, item_next / RTU);
          ask_ahead((mat == 0 ? a.w0 : a.w1) + (uint64_t)tn.slot * a.slice_bytes, item_rows0(item_next) + m);
        }
        if (!ok || it + kDecGroups >= KT) break;
        if (it + 2 * kDecGroups < KT) fetch(0, it + 2 * kDecGroups);
        stage_step(1, it + kDecGroups);
      }
      }
      if (is_wide(t.count)) {
        // Both buffers: the next item's MMAs wait for this epilogue, so these warps take four fifths of it.
        if (ok) ok = mbar_wait(acc_full(0), use0 & 1, abort, a.error);
        if (ok) ok = mbar_wait(acc_full(1), use1 & 1, abort, a.error);
        if (ok) {
          tc_fence_after();
          drain(t, r0, 0, kTileN, warp / 4, kDW / 4 + 1);
          tc_fence_before();
          __syncwarp();
          if (lane == 0) arrive_lead(acc_empty_wide_lead, acc_empty_wide);
        }
        use0++, use1++, wides++;
      } else {
        use_inc(next_buf), next_buf ^= 1;
      }
    }
  } else if (warp < kDW + kEW) {
    // Epilogue warps: warp w reads TMEM lanes 32 (w % 4) .., its quarter of the weight rows.
    uint32_t li = 0;
    for (uint32_t rnd = 0, item; (item = item_at(rnd)) != kNoItem && ok; rnd++, li++) {
      const ItemTile t = item_tile(a, item / RTU);
      const uint32_t r0 = item_rows0(item);
      if (is_wide(t.count)) {
        if (ok) ok = mbar_wait(acc_full(0), use0 & 1, abort, a.error);
        if (ok) ok = mbar_wait(acc_full(1), use1 & 1, abort, a.error);
        if (!ok) break;
        tc_fence_after();
        drain(t, r0, 0, kTileN, kDW / 4, kDW / 4 + 1);
        tc_fence_before();
        __syncwarp();
        if (lane == 0) arrive_lead(acc_empty_lead(0), acc_empty(0)), arrive_lead(acc_empty_lead(1), acc_empty(1));
        use0++, use1++, wides++;
      } else {
        const uint32_t b = next_buf;
        ok = mbar_wait(acc_full(b), use_of(b) & 1, abort, a.error);
        if (!ok) break;
        tc_fence_after();
        drain(t, r0, b * kTileN, b * kTileN + kTileN / 2, 0, 1);
        tc_fence_before();
        __syncwarp();
        if (lane == 0) arrive_lead(acc_empty_lead(b), acc_empty(b));
        use_inc(b), next_buf ^= 1;
      }
    }
  } else if (warp == kCopyWarp) {
    if (a.gather_rows) {
      // The copy warp, gathering: the tile's rows are scattered over the activations (row r of the expert order is row
      // gather_rows[r] of the map's tensor) and a copy brings four of them: up to 32 copies a stage for a pair's CTA (one
      // a lane), 64 for a single CTA (two a lane). A lane keeps its row indices for the whole item. Rows past the
      // tile's count repeat its last row; their columns of the result are dropped.
      constexpr uint32_t kPerLane = PAIR ? 1 : 2;
      uint32_t li = 0;
      for (uint32_t rnd = 0, item; (item = item_at(rnd)) != kNoItem && ok; rnd++, li++) {
        const ItemTile t = item_tile(a, item / RTU);
        const uint32_t half = ((t.count + 15) & ~15u) / 2;
        const uint32_t mine = PAIR ? half : t.count, first_row = PAIR ? rank * half : 0;
        const uint32_t ncopies = (mine + 3) / 4;
        uint32_t idx[4 * kPerLane];
#pragma unroll
        for (uint32_t j = 0; j < 4 * kPerLane; j++) {
          const uint32_t r = first_row + 4 * (lane + 32 * (j / 4)) + j % 4;
          idx[j] = a.gather_rows[t.start + min(r, t.count - 1)];
        }
        for (uint32_t it = 0; it < KT && ok; it++) {
          const uint32_t g = li * KT + it, s = g % S, use_s = g / S;
          const uint32_t bar = PAIR ? full_lead(s) : full_bar(s);
          if (lane == 0) {
            if (use_s > 0) ok = mbar_wait(empty_bar(s), (use_s - 1) & 1, abort, a.error);
            if (ok) {
              if constexpr (PAIR)
                mbar_arrive_expect_cluster(bar, ncopies * 4 * kTileK * 2);
              else
                mbar_arrive_expect(bar, ncopies * 4 * kTileK * 2);
            }
          }
          ok = __shfl_sync(0xffffffffu, ok, 0);
          if (!ok) break;
          const uint32_t xt = smem_u32(smem + s * SM::kStageBytes) + NMAT * SM::kWBytes;
#pragma unroll
          for (uint32_t c = 0; c < kPerLane; c++) {
            const uint32_t copy = lane + 32 * c;
            if (copy < ncopies) {
              if constexpr (PAIR)
                tma_gather4_rows_pair(xt + copy * 4 * kTileK * 2, &act_map, it * kTileK, idx[4 * c], idx[4 * c + 1], idx[4 * c + 2], idx[4 * c + 3], bar);
              else
                tma_gather4_rows(xt + copy * 4 * kTileK * 2, &act_map, it * kTileK, idx[4 * c], idx[4 * c + 1], idx[4 * c + 2], idx[4 * c + 3], bar);
            }
          }
        }
      }
      if (!ok && lane == 0) {
        const long long t0 = clock64();
        while (clock64() - t0 < 400000) {
        }
      }
      __syncwarp();
    } else if (lane == 0) {
      // The copy thread: per stage, the 64 values of the tile's rows, 64 rows a copy, in the swizzled layout. A copy may
      // run past the tile's rows into the next expert's, or past the tensor (zeros): those columns of the result are dropped.
      uint32_t li = 0;
      for (uint32_t rnd = 0, item; (item = item_at(rnd)) != kNoItem && ok; rnd++, li++) {
        const ItemTile t = item_tile(a, item / RTU);
        // A CTA of a pair brings its half of the rows the instruction takes (the rows rounded up to 16): the first
        // CTA the first half.
        const uint32_t half = ((t.count + 15) & ~15u) / 2;
        const uint32_t mine = PAIR ? half : t.count, row0 = t.start + (PAIR ? rank * half : 0);
        const uint32_t nbox = (mine + kTileBoxRows - 1) / kTileBoxRows;
        for (uint32_t it = 0; it < KT && ok; it++) {
          const uint32_t g = li * KT + it, s = g % S, use_s = g / S;
          if (use_s > 0) ok = mbar_wait(empty_bar(s), (use_s - 1) & 1, abort, a.error);
          if (!ok) break;
          const uint32_t xt = smem_u32(smem + s * SM::kStageBytes) + NMAT * SM::kWBytes;
          if constexpr (PAIR) {
            mbar_arrive_expect_cluster(full_lead(s), nbox * kTileBoxRows * kTileK * 2);
            for (uint32_t i = 0; i < nbox; i++)
              tma_load_rows_pair(xt + i * kTileBoxRows * kTileK * 2, &act_map, it * kTileK, row0 + i * kTileBoxRows, full_lead(s));
          } else {
            mbar_arrive_expect(full_bar(s), nbox * kTileBoxRows * kTileK * 2);
            for (uint32_t i = 0; i < nbox; i++)
              tma_load_rows(xt + i * kTileBoxRows * kTileK * 2, &act_map, it * kTileK, row0 + i * kTileBoxRows, full_bar(s));
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
  } else if (warp == kQuantWarp) {
    if (quants_by_copy(QT) && lane == 0) {
    // The quants' copy thread (a warp of its own: sharing a warp with the MMA thread cost the tile kernels 8 %): a quant slot, one stage per decode group for every weight row of the item, as soon
    // as the decode warps have read the slot's last contents; it runs ahead of the stages by the ring's two slots.
    uint32_t li = 0;
    for (uint32_t rnd = 0, item; (item = item_at(rnd)) != kNoItem && ok; rnd++, li++) {
      const ItemTile t = item_tile(a, item / RTU);
      for (uint32_t j = 0; j < KT / kDecGroups && ok; j++) {
        const uint32_t qn = li * (KT / kDecGroups) + j, qb = qn % SM::kQSlots, use_q = qn / SM::kQSlots;
        if (use_q > 0) ok = mbar_wait(q_empty(qb), (use_q - 1) & 1, abort, a.error);
        if (!ok) break;
        const uint32_t dst = smem_u32(smem + SM::kQuants + qb * SM::kQSlotBytes);
        mbar_arrive_expect(q_full(qb), SM::kQSlotBytes);
        for (uint32_t mt = 0; mt < (uint32_t)NMAT; mt++)
          tma_load_quants(dst + mt * SM::kQMatBytes, &a.qmap[mt], j * SM::kQRowBytes, item_rows0(item), t.slot, q_full(qb));
      }
    }
    if (!ok) {
      const long long t0 = clock64();
      while (clock64() - t0 < 400000) {
      }
    }
    }
  } else if (lane == 0 && rank == 0) {
    // The MMA thread (of a pair's first CTA): per stage, four K steps of 16 for each matrix; the commit frees the stage
    // when they are done, in both CTAs of a pair.
    auto wait_lead = [&](uint32_t bar, uint32_t parity) { return mbar_wait(bar, parity, abort, a.error); };
    auto mma = [&](uint32_t d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t acc) {
      if constexpr (PAIR)
        mma_f16_pair(d, da, db, idesc, acc);
      else
        mma_f16(d, da, db, idesc, acc);
    };
    auto commit = [&](uint32_t bar) {
      if constexpr (PAIR)
        mma_commit_pair(bar, 3);
      else
        mma_commit(bar);
    };
    uint32_t li = 0;
    bool after_wide = false;
    for (uint32_t rnd = 0, item; (item = item_at(rnd)) != kNoItem && ok; rnd++, li++) {
      const ItemTile t = item_tile(a, item / RTU);
      const uint32_t idesc = instr_desc((t.count + 15) & ~15u, PAIR ? 2 * kTileM : kTileM);
      const bool wide = is_wide(t.count);
      const uint32_t b = next_buf, colg = wide ? 0 : b * kTileN, colu = wide ? kTileN : colg + kTileN / 2;
      // The buffers this item writes must have been read: by the epilogue warps, and after a two-buffer item by the
      // decode warps too.
      if (after_wide) ok = wait_lead(acc_empty_wide, (wides - 1) & 1);
      after_wide = false;
      for (uint32_t bb = 0; bb < 2 && ok; bb++)
        if ((wide || bb == b) && use_of(bb) > 0) ok = wait_lead(acc_empty(bb), (use_of(bb) - 1) & 1);
      for (uint32_t it = 0; it < KT && ok; it++) {
        const uint32_t g = li * KT + it, s = g % S;
        ok = wait_lead(full_bar(s), (g / S) & 1);
        if (!ok) break;
        tc_fence_after();
        const uint32_t stage = smem_u32(smem + s * SM::kStageBytes), xt = stage + NMAT * SM::kWBytes;
#pragma unroll
        for (uint32_t k = 0; k < kTileK / 16; k++) {
          const uint64_t db = smem_desc_sw128(xt + 32 * k);
          mma(tmem_base + colg, smem_desc(stage + 2 * k * kLbo), db, idesc, (it | k) != 0);
          if constexpr (NMAT == 2) mma(tmem_base + colu, smem_desc(stage + SM::kWBytes + 2 * k * kLbo), db, idesc, (it | k) != 0);
        }
        commit(empty_bar(s));
      }
      if (!ok) break;
      if (wide) {
        commit(acc_full(0)), commit(acc_full(1));
        use0++, use1++, wides++, after_wide = true;
      } else {
        commit(acc_full(b));
        use_inc(b), next_buf ^= 1;
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  // Neither CTA of a pair may leave (or free tensor memory) while the other may still read its shared memory or write
  // its tensor memory.
  if constexpr (PAIR) cluster_sync();
  if (warp == kMmaWarp) {
    __syncwarp();
    tc_fence_after();
    if constexpr (PAIR)
      tmem_free_pair(tmem_base, kCols);
    else
      tmem_free(tmem_base, kCols);
  }
}

// act_map: the activation rows, f16 [rows][a.K] in the order of the tiles (tensor_map.h).
struct LaunchCtx;
template <int QT, int NMAT>
cudaError_t launch_expert_tiles(const ExpertTilesArgs &a, const CUtensorMap &act_map, uint32_t max_tiles, const uint32_t *grid_global,
                                const LaunchCtx &ctx, cudaStream_t st);

}  // namespace moe
