// Tensor maps for the bulk-tensor (TMA) copies of the tile kernels' activation rows.
#pragma once

#include <cuda.h>

#include <cstdint>

namespace moe {

constexpr uint32_t kMapBoxRows = 64;  // rows one copy brings: a tile of n rows takes ceil(n / 64) copies a stage

// A map over f16 rows [rows][K] in device memory (base 16-byte aligned, K a multiple of 64) whose copies bring a box of
// 64 values x 64 rows into shared memory with the 128-byte swizzle, the layout the tensor core reads K-major operands
// in. Rows past `rows` read as zero. Throws CudaFailure when the driver refuses the map.
// box_rows: the rows one copy brings, at most 256 (the tensor must be at least that high).
CUtensorMap make_rows_map(const void *base, uint64_t rows, uint32_t K, uint32_t box_rows = kMapBoxRows);

// A map over the quants run of a weight matrix in the runs layout, for types whose rows' quants are one run of
// row_bytes bytes a row (Q4_K: K / 2): bytes [rows][row_bytes] per expert slot, the slots slice_bytes apart. A copy
// brings box_bytes of 128 rows of one slot, swizzled by box_bytes (64 or 128), so that the decode warps' 16-byte reads
// of neighbouring rows fall on different banks.
CUtensorMap make_quants_map(const void *base, uint32_t row_bytes, uint32_t rows, uint32_t nslots, uint64_t slice_bytes, uint32_t box_bytes);

}  // namespace moe
