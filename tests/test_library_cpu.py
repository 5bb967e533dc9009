"""Without a GPU: the C-ABI library loads, exports every symbol include/moe_layer.h declares, its struct layouts
match the Python mirror (the reference's tests/host/test_abi.py:31-45 in kind), and the host repack is the
permutation the oracle's is (core/tests/quant_test.cpp:76-81)."""
import ctypes
import itertools
import os
import re

import numpy as np
import pytest

from c0ven_b200 import _lib, synth
from oracle import oracle as O

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_every_declared_symbol_is_exported():
    header = open(os.path.join(ROOT, "include", "moe_layer.h")).read()
    declared = set(re.findall(r"MOE_API\s+[\w\s\*]+?\b(moe_\w+)\s*\(", header))
    assert declared == set(_lib.SYMBOLS)
    L = _lib.lib()
    for name in declared:
        assert hasattr(L, name), name


def test_struct_layouts_match_the_library():
    rows = _lib.abi_layout()
    for name, struct in _lib.STRUCTS.items():
        assert (name, 0, ctypes.sizeof(struct)) in rows
        fields = {r[0] for r in rows if r[0].startswith(name + ".")}
        assert fields == {f"{name}.{f[0]}" for f in struct._fields_}
        for f, _ in struct._fields_:
            d = getattr(struct, f)
            assert (f"{name}.{f}", d.offset, d.size) in rows
        spans = sorted((o, o + s) for n, o, s in rows if n.startswith(name + "."))
        for (_, end), (start, _) in itertools.pairwise(spans):
            assert end <= start
    assert ctypes.sizeof(_lib.Tile) == 16  # shared/moe_tile.h:18
    assert ctypes.sizeof(_lib.Config) == 68 and ctypes.sizeof(_lib.Weights) == 72 and ctypes.sizeof(_lib.Stats) == 72


@pytest.mark.parametrize("t", [synth.Q8_0, synth.Q4_K, synth.Q6_K, synth.IQ3_S, synth.IQ4_NL, synth.IQ4_XS, synth.IQ3_XXS, synth.IQ2_S, synth.Q2_0])
def test_host_repack_is_a_permutation_in_run_order(t):
    rng = np.random.default_rng(t)
    n = 256
    blocks = synth.random_blocks(t, n, rng)
    runs = np.empty_like(blocks)
    L = _lib.lib()
    assert L.moe_to_runs(t, blocks.ctypes.data, n, runs.ctypes.data) == _lib.MOE_OK
    assert np.array_equal(np.sort(runs.reshape(-1)), np.sort(blocks.reshape(-1)))
    if t != synth.Q4_K:  # Q4_K keeps d, dmin and the scales as one 16-byte piece; the others are the reference's runs
        assert np.array_equal(runs.reshape(-1), O.to_runs(t, blocks).reshape(-1))
    else:
        assert np.array_equal(runs.reshape(-1)[:n * 128].reshape(n, 128), blocks[:, 16:])
        assert np.array_equal(runs.reshape(-1)[n * 128:].reshape(n, 16), blocks[:, :16])
    back = np.empty_like(blocks)
    assert L.moe_from_runs(t, runs.ctypes.data, n, back.ctypes.data) == _lib.MOE_OK
    assert np.array_equal(back, blocks)
    assert L.moe_to_runs(3, blocks.ctypes.data, n, runs.ctypes.data) == _lib.MOE_BAD_ARGUMENT


def test_create_fails_loudly_without_a_gpu_or_with_a_bad_shape():
    import torch

    from c0ven_b200 import MoEError, MoELayer

    layer = synth.make_layer(256, 256, 32, 4)
    bad = dict(layer, n_experts=33)
    with pytest.raises(MoEError) as e:
        MoELayer(bad)
    assert e.value.status == _lib.MOE_BAD_ARGUMENT
    if not torch.cuda.is_available():
        with pytest.raises(MoEError) as e:
            MoELayer(layer)
        assert e.value.status == _lib.MOE_ERROR  # no device: an error, never another path
