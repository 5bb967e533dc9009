"""The engine ABI without a GPU: libengine.so loads and exports the reference's twenty engine_* symbols and nothing
else of the library's; its engine_abi_layout equals, row for row, the layout a C compiler gives the reference's own
header (tests/golden/engine_abi_layout.json, made from include/engine_api.h by tests/golden/make_engine_abi_golden.py;
the reference holds itself to the same table: tests/host/test_abi.py:12-56); the ctypes mirror agrees with both; and
calls that need no GPU answer as the header says."""
import ctypes
import itertools
import json
import os
import subprocess

import pytest

from c0ven_b200 import engine as E

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
GOLDEN = json.load(open(os.path.join(ROOT, "tests", "golden", "engine_abi_layout.json")))["rows"]


def test_library_exports_the_twenty_symbols_and_only_the_engines():
    L = E.lib()
    for name in E.SYMBOLS:
        assert hasattr(L, name), name
    assert len(E.SYMBOLS) == 20
    out = subprocess.run(["nm", "-D", "--defined-only", E.LIB_PATH], capture_output=True, text=True, check=True).stdout
    exported = {ln.split()[-1] for ln in out.splitlines() if " T " in ln}
    assert set(E.SYMBOLS) <= exported
    assert all(s.startswith("engine_") for s in exported), sorted(s for s in exported if not s.startswith("engine_"))
    header = open(os.path.join(ROOT, "include", "engine_abi.h")).read()
    import re
    declared = set(re.findall(r"ENGINE_API\s+[\w\s\*]+?\b(engine_\w+)\s*\(", header))
    assert declared == exported


def test_layout_is_the_reference_headers_row_for_row():
    mine = sorted(E.abi_layout())
    want = sorted((n, o, s) for n, o, s in GOLDEN)
    assert mine == want


def test_ctypes_mirror_matches_the_library():
    rows = E.abi_layout()
    for name, struct in E.STRUCTS.items():
        assert (name, 0, ctypes.sizeof(struct)) in rows
        fields = {r[0] for r in rows if r[0].startswith(name + ".")}
        assert fields == {f"{name}.{f[0]}" for f in struct._fields_}
        for f, *_ in struct._fields_:
            d = getattr(struct, f)
            assert (f"{name}.{f}", d.offset, d.size) in rows
        spans = sorted((o, o + s) for n, o, s in rows if n.startswith(name + "."))
        for (_, end), (start, _) in itertools.pairwise(spans):
            assert end <= start, name
    # the sizes the reference's own test names (tests/host/test_abi.py:29-45)
    sizes = {n: ctypes.sizeof(s) for n, s in E.STRUCTS.items()}
    assert sizes["engine_config"] == 96 and sizes["engine_info"] == 176 and sizes["engine_card"] == 120
    assert sizes["engine_settings"] == 80 and sizes["engine_page_change"] == 20 and sizes["engine_event"] == 16
    assert sizes["engine_timing"] == 32 and sizes["engine_image"] == 24 and sizes["engine_stats"] == 8 * 62 and sizes["engine_slot_stats"] == 8 * 7
    assert sizes["engine_step_plan"] == 4 + 4 * E.MAX_STEP_SLOTS + 4 + 8 * E.MAX_PROMPT_PIECES + 4 + 4 + 8 + 4 + 4


def test_open_refuses_what_it_cannot_load():
    L = E.lib()
    h = ctypes.c_void_p()
    assert L.engine_open(None, None, ctypes.byref(h)) == E.BAD_ARGUMENT
    cfg = E.Config(model_path=b"/nonexistent/model.gguf")
    st = L.engine_open(ctypes.byref(cfg), None, ctypes.byref(h))
    assert st in (E.ERROR, E.BAD_ARGUMENT) and not h.value
    assert len(L.engine_last_error(None)) > 0
    assert L.engine_queue_stuck() == 0
    assert L.engine_poll(None, None, 0, None) == E.BAD_ARGUMENT
