"""The block formats' sizes, fields and runs layout, and the pack's tile record, held to the reference's own headers
(shared/quant.h:36-177, shared/moe_tile.h:9-18) compiled as they are into oracle/_ref/libref_layout.so
(oracle/ref_layout.cpp; `make -C oracle REFERENCE=<the reference's root> ref`). Skipped where that library was not built."""
import ctypes as C
import os

import numpy as np
import pytest

from c0ven_b200 import _lib, synth

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF_SO = os.path.join(ROOT, "oracle", "_ref", "libref_layout.so")
TYPES = [synth.Q8_0, synth.Q4_K, synth.Q6_K, synth.IQ3_S, synth.IQ4_NL, synth.IQ4_XS, synth.IQ3_XXS, synth.IQ2_S, synth.Q2_0]

pytestmark = pytest.mark.skipif(not os.path.exists(REF_SO), reason="oracle/_ref is built only where the reference's tree is")


@pytest.fixture(scope="module")
def ref():
    R = C.CDLL(REF_SO)
    R.ref_quant_run_offset.restype = C.c_uint64
    R.ref_quant_run_offset.argtypes = [C.c_uint32, C.c_uint32, C.c_uint64]
    return R


def test_type_ids_and_block_sizes_are_the_references(ref):
    assert synth.Q2_0 == ref.ref_qt_q2_0()
    for t in TYPES:
        assert synth.BLOCK_VALUES[t] == ref.ref_quant_block_values(t), t
        assert synth.BLOCK_BYTES[t] == ref.ref_quant_block_bytes(t), t


@pytest.mark.parametrize("t", TYPES)
def test_the_librarys_runs_are_the_references_runs(ref, t):
    """moe_to_runs against the permutation the reference's field table and run offsets give. Q4_K here keeps its d, dmin
    and scales together as one 16-byte piece a block after the quants' run; its quants' run is the reference's."""
    n = 96
    blocks = synth.random_blocks(t, n, np.random.default_rng(100 + t))
    want = np.empty(blocks.size, dtype=np.uint8)
    covered = 0
    for f in range(ref.ref_quant_nfields(t)):
        off, size, run = ref.ref_quant_field_offset(t, f), ref.ref_quant_field_size(t, f), ref.ref_quant_run_offset(t, f, n)
        want[run:run + n * size] = blocks[:, off:off + size].reshape(-1)
        covered += size
    assert covered == synth.BLOCK_BYTES[t]          # the fields tile the block
    got = np.empty_like(blocks)
    assert _lib.lib().moe_to_runs(t, blocks.ctypes.data, n, got.ctypes.data) == _lib.MOE_OK
    if t == synth.Q4_K:
        assert ref.ref_quant_run_offset(t, 1, n) == n * 128
        assert np.array_equal(got.reshape(-1)[:n * 128], want[:n * 128])
    else:
        assert np.array_equal(got.reshape(-1), want)


def test_the_tile_record_is_the_references(ref):
    out = (C.c_uint32 * 5)()
    ref.ref_moe_tile_layout(out)
    assert C.sizeof(_lib.Tile) == out[0]
    assert [getattr(_lib.Tile, f).offset for f in ("expert", "slot", "start", "count")] == list(out[1:])
    # A run of 200 rows of one expert: the oracle's pack (which the GPU's is held to bit for bit) cuts it into tiles of
    # the reference's MOE_TILE rows.
    from oracle import oracle as O

    tiles = O.pack(np.zeros(200, dtype=np.int32), 4)[3]
    assert [int(c) for c in tiles[:, 3]] == [ref.ref_moe_tile_rows()] * 3 + [200 - 3 * ref.ref_moe_tile_rows()]
    assert ref.ref_moe_group_max() == 8              # the most rows of a group of k_expert_rows (route_kernels.cuh: kGroupMax)
