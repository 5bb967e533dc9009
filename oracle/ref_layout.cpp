// Test infrastructure, like everything under oracle/: nothing the product runs links, loads or calls this.
//
// The reference's own shared headers, compiled where they lie (shared/quant.h: the block formats' sizes, fields and
// the runs layout; shared/moe_tile.h: the pack's tile and group records) and given C names, so that the tests can
// hold this repository's tables (c0ven_b200/csrc/formats.h, include/moe_layer.h) to the reference's code rather than
// to a restatement of it. Built by oracle/Makefile's `ref` target into oracle/_ref/libref_layout.so when the
// reference's tree is at hand (make REFERENCE=<its root> ref); the tests that use it skip without it.
#include <cstddef>
#include <cstdint>

#include "moe_tile.h"
#include "quant.h"

extern "C" {
uint32_t ref_quant_block_values(uint32_t t) { return quant_block_values(t); }
uint32_t ref_quant_block_bytes(uint32_t t) { return quant_block_bytes(t); }
uint32_t ref_quant_nfields(uint32_t t) { return quant_nfields(t); }
uint32_t ref_quant_field_offset(uint32_t t, uint32_t f) { return quant_field_offset(t, f); }
uint32_t ref_quant_field_size(uint32_t t, uint32_t f) { return quant_field_size(t, f); }
uint64_t ref_quant_run_offset(uint32_t t, uint32_t f, uint64_t n) { return quant_run_offset(t, f, n); }
uint32_t ref_qt_q2_0(void) { return QT_Q2_0; }
uint32_t ref_moe_tile_rows(void) { return MOE_TILE; }
uint32_t ref_moe_group_max(void) { return MOE_GROUP_MAX; }
// (size, offsets of expert, slot, start, count)
void ref_moe_tile_layout(uint32_t out[5]) {
  out[0] = sizeof(MoeTile), out[1] = offsetof(MoeTile, expert), out[2] = offsetof(MoeTile, slot), out[3] = offsetof(MoeTile, start),
  out[4] = offsetof(MoeTile, count);
}
}
