// The GGUF block formats the layer reads and the "runs" layout the GPU holds them in: a slice of n blocks is one run
// per field, the quants first and the f16 scales last, field f of block k at run_offset(f, n) + k * field_size(f).
// The formats and the run order are the reference's (shared/quant.h:36-176; docs/spec/QUANT_FORMATS.md, "Wide loads"),
// but for Q4_K, whose d, dmin and packed scales stay together as the block's first 16 bytes, so one 128-bit load brings them;
// the layout is a permutation of the file's bytes, so an expert costs the bytes it has in the file.
// IQ4_NL (y = d * table[nibble], blocks of 32) and IQ4_XS (y = d * (ls - 32) * table[nibble], 256 values with a 6-bit
// scale per 32) share ggml's 16-entry table of signed bytes (docs/spec/QUANT_FORMATS.md:213-247); they are the types of
// the reference file's down and (in one layer) gate/up experts.
// Q2_0 (the reference's fork of ggml, type 42: y = (q - 1) * d, 64 values a block, QUANT_FORMATS.md:251-270) has two
// bits a value and one scale.
// IQ3_XXS and IQ2_S (QUANT_FORMATS.md:115-173) are codebook types like IQ3_S: groups of 4 or 8 values are entries of a
// table (256 of 4 bytes; 1024 of 8), with sign bits and a 4-bit scale beside them.
#pragma once

#include <cstdint>

#if defined(__CUDACC__)
#define FMT_HD __host__ __device__
#else
#define FMT_HD
#endif

namespace moe {

enum : uint32_t { QT_Q8_0 = 8, QT_Q4_K = 12, QT_Q6_K = 14, QT_IQ3_XXS = 18, QT_IQ4_NL = 20, QT_IQ3_S = 21, QT_IQ2_S = 22, QT_IQ4_XS = 23, QT_Q2_0 = 42 };

FMT_HD constexpr uint32_t block_values(uint32_t t) {
  return t == QT_Q2_0 ? 64u : (t == QT_Q8_0 || t == QT_IQ4_NL) ? 32u : (t == QT_Q4_K || t == QT_Q6_K || t == QT_IQ3_S || t == QT_IQ4_XS || t == QT_IQ3_XXS || t == QT_IQ2_S) ? 256u : 0u;
}
FMT_HD constexpr uint32_t block_bytes(uint32_t t) {
  return t == QT_Q8_0 ? 34u : t == QT_Q4_K ? 144u : t == QT_Q6_K ? 210u : t == QT_IQ3_S ? 110u : t == QT_IQ4_NL ? 18u : t == QT_IQ4_XS ? 136u : t == QT_IQ3_XXS ? 98u : t == QT_IQ2_S ? 82u : t == QT_Q2_0 ? 18u : 0u;
}
FMT_HD constexpr bool type_known(uint32_t t) { return block_bytes(t) != 0; }
// Whether the type's dot takes activations as q8_K (256 values, f32 scale, sums of 16) rather than q8_0 (32 values,
// f16 scale): docs/spec/MODEL_LAYER.md, section 6.
FMT_HD constexpr bool act_is_q8k(uint32_t t) { return t != QT_Q8_0 && t != QT_IQ4_NL && t != QT_Q2_0; }
FMT_HD constexpr uint64_t row_bytes(uint32_t t, uint64_t n) { return n / block_values(t) * block_bytes(t); }

// Types whose values come from a codebook the kernels keep in shared memory: its words, and where it starts in the
// layer's one table of all of them on the device (IQ3_S 512 words, IQ3_XXS 256, IQ2_S 2048: two words an entry).
FMT_HD constexpr uint32_t grid_words(uint32_t t) { return t == QT_IQ3_S ? 512u : t == QT_IQ3_XXS ? 256u : t == QT_IQ2_S ? 2048u : 0u; }
FMT_HD constexpr uint32_t grid_offset(uint32_t t) { return t == QT_IQ3_XXS ? 512u : t == QT_IQ2_S ? 768u : 0u; }
constexpr uint32_t kGridWordsAll = 512 + 256 + 2048;

struct Field {
  uint32_t offset, size;
};
FMT_HD constexpr uint32_t nfields(uint32_t t) {
  return t == QT_Q8_0 ? 2u : t == QT_Q4_K ? 2u : t == QT_Q6_K ? 4u : t == QT_IQ3_S ? 5u : t == QT_IQ4_NL ? 2u : t == QT_IQ4_XS ? 4u : t == QT_IQ3_XXS ? 3u : t == QT_IQ2_S ? 5u : t == QT_Q2_0 ? 2u : 0u;
}
// Field f of type t, in run order.
FMT_HD constexpr Field field(uint32_t t, uint32_t f) {
  switch (t) {
    case QT_Q8_0: return f == 0 ? Field{2, 32} : Field{0, 2};                                                  // qs, d
    case QT_Q4_K: return f == 0 ? Field{16, 128} : Field{0, 16};  // qs; then d, dmin and the scales as one 16-byte piece, one load
    case QT_Q6_K: return f == 0 ? Field{0, 128} : f == 1 ? Field{128, 64} : f == 2 ? Field{192, 16} : Field{208, 2};  // ql, qh, scales, d
    case QT_IQ3_S:
      return f == 0 ? Field{2, 64} : f == 1 ? Field{74, 32} : f == 2 ? Field{66, 8} : f == 3 ? Field{106, 4} : Field{0, 2};  // qs, signs, qh, scales, d
    case QT_Q2_0:  // qs, d: 64 values in 16 bytes
    case QT_IQ4_NL: return f == 0 ? Field{2, 16} : Field{0, 2};                                                // qs, d
    case QT_IQ4_XS: return f == 0 ? Field{8, 128} : f == 1 ? Field{4, 4} : f == 2 ? Field{2, 2} : Field{0, 2};   // qs, scales_l, scales_h, d
    case QT_IQ3_XXS: return f == 0 ? Field{2, 64} : f == 1 ? Field{66, 32} : Field{0, 2};                       // grid indices, scale-and-sign words, d
    case QT_IQ2_S:
      return f == 0 ? Field{2, 32} : f == 1 ? Field{34, 32} : f == 2 ? Field{66, 8} : f == 3 ? Field{74, 8} : Field{0, 2};  // index low bits, signs, qh, scales, d
    default: return Field{0, 0};
  }
}
FMT_HD constexpr uint64_t run_offset(uint32_t t, uint32_t f, uint64_t n) {
  uint64_t off = 0;
  for (uint32_t g = 0; g < f; g++) off += field(t, g).size;
  return off * n;
}

// Host repack, threaded (runs.cpp). Both are permutations of the slice's bytes.
void to_runs(uint32_t type, const uint8_t *file_blocks, uint64_t nblocks, uint8_t *dst);
void from_runs(uint32_t type, const uint8_t *runs, uint64_t nblocks, uint8_t *dst);
// nslices slices of nblocks each, one after another, on up to `threads` threads.
void to_runs_slices(uint32_t type, const uint8_t *file_blocks, uint64_t nblocks, uint64_t nslices, uint8_t *dst,
                    unsigned threads);

}  // namespace moe
