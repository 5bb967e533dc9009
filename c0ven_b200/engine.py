"""ctypes binding of libengine.so, the library behind include/engine_abi.h: the structs of the reference's engine ABI
mirrored by hand, as its own control plane mirrors them (engine/api/abi.py) and binds its core (engine/api/native.py:227),
and a small Engine class over the calls. The library is required; nothing here stands in for it."""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libengine.so")

OK, ERROR, BAD_ARGUMENT, BUSY, TIMEOUT = range(5)
EVENT_TOKEN, EVENT_PROMPT, EVENT_DONE, EVENT_STEP, EVENT_ERROR, EVENT_STALLED = range(1, 7)
TIMING_PROMPT, TIMING_DECODE = 1, 2
MAX_STOP, MAX_STEP_SLOTS, MAX_PROMPT_PIECES, NO_PAGE = 8, 8, 4, 0xFFFFFFFF
CONFIG_PROMPT_SET = 2

SYMBOLS = ("engine_open", "engine_admit", "engine_admit_images", "engine_release", "engine_submit", "engine_poll", "engine_wait",
           "engine_checkpoint", "engine_restore", "engine_drop", "engine_read_timing", "engine_read_stats", "engine_read_slot_stats",
           "engine_sleep", "engine_wake", "engine_last_error", "engine_close", "engine_queue_stuck", "engine_cards", "engine_abi_layout")

u32, i32, u64, f32, f64 = C.c_uint32, C.c_int32, C.c_uint64, C.c_float, C.c_double


class Config(C.Structure):
    _fields_ = [("model_path", C.c_char_p), ("slots", u32), ("max_ctx", u32), ("max_cards", u32), ("experts_per_layer", i32),
                ("cpu_threads", u32), ("flags", u32), ("reserve_bytes", u64), ("prompt_chunk", u32), ("checkpoints", u32),
                ("routing_profile", C.c_char_p), ("mtp_dir", C.c_char_p), ("draft_max", u32), ("draft_min_p", f32),
                ("vision_path", C.c_char_p), ("kv_pages", u32), ("kv_resident_cells", u32), ("ngram_huge_bytes", u64)]


class Info(C.Structure):
    _fields_ = [("api_version", u32), ("cards", u32), ("slots", u32), ("max_ctx", u32), ("experts_per_layer", u32), ("vocab", u32),
                ("device_bytes", u64 * 2), ("arena_bytes", u64), ("load_seconds", f64), ("prompt_chunk", u32), ("checkpoints", u32),
                ("max_step_rows", u32), ("drafting", u32), ("image_tokens_max", u32), ("kv_pages", u32), ("pages_per_slot", u32),
                ("host_read_bytes_per_s", f64), ("loader_threads", u32), ("ngram_in_ram", u32), ("loader_bytes_per_s", f64),
                ("ngram_read_us", f64), ("copy_bytes_per_s", f64 * 2), ("expert_budget", u64 * 2), ("fetch_rows", u32),
                ("decode_weight", u32), ("ngram_cache_rows", u64), ("ngram_huge_bytes", u64)]


class Settings(C.Structure):
    _fields_ = [("temperature", f32), ("top_k", u32), ("top_p", f32), ("max_tokens", u32), ("seed", u64), ("n_stop", u32),
                ("stop", i32 * MAX_STOP), ("min_p", f32), ("penalty_last_n", u32), ("penalty_repeat", f32), ("penalty_freq", f32),
                ("penalty_present", f32)]


class PageChange(C.Structure):
    _fields_ = [("slot", u32), ("logical", u32), ("page", u32), ("source", u32), ("cells", u32)]


class PromptPiece(C.Structure):
    _fields_ = [("slot", u32), ("tokens", u32)]


class StepPlan(C.Structure):
    _fields_ = [("nslots", u32), ("slots", u32 * MAX_STEP_SLOTS), ("npieces", u32), ("pieces", PromptPiece * MAX_PROMPT_PIECES),
                ("npages", u32), ("pages", C.POINTER(PageChange)), ("kv_free", u32), ("window_rows", u32)]


class Event(C.Structure):
    _fields_ = [("kind", u32), ("slot", u32), ("token", i32), ("value", u32)]


class Timing(C.Structure):
    _fields_ = [("kind", u32), ("plan", u32), ("rows", u32), ("misses", u32), ("start_ns", u64), ("end_ns", u64)]


_STATS = ("up_ns plans busy_ns prompt_chunks prompt_rows prompt_ns window_pieces window_rows window_ns steps step_rows step_ns step_misses "
          "step_layers_missed undrafted_steps rounds round_rows round_ns round_misses round_layers_missed layer_runs layer_drafts "
          "layer_accepted layer_ns lookup_runs lookup_drafts lookup_accepted lookup_ns swap_rounds swaps swap_ns stalls checkpoints_taken "
          "restores ngram_rows ngram_hits ngram_reads experts_cached experts_floor idle_rounds reading_steps reading_rounds draft_passes "
          "draft_ns layer_drafts_1 layer_drafts_2 layer_drafts_3 layer_drafts_4 layer_drafts_5 layer_drafts_6 layer_drafts_7 "
          "layer_accepted_1 layer_accepted_2 layer_accepted_3 layer_accepted_4 layer_accepted_5 layer_accepted_6 layer_accepted_7 "
          "layer_stop_max layer_stop_share layer_stop_p layer_stop_choice").split()


class Stats(C.Structure):
    _fields_ = [(n, u64) for n in _STATS]


class SlotStats(C.Structure):
    _fields_ = [(n, u64) for n in ("steps", "rounds", "drafts", "accepted", "lookup_rounds", "lookup_drafts", "lookup_accepted")]


class Image(C.Structure):
    _fields_ = [("first", u32), ("grid_h", u32), ("grid_w", u32), ("frames", u32), ("pixels", C.c_void_p)]


class Card(C.Structure):
    _fields_ = [("name", C.c_char * 64), ("pci", C.c_char * 16), ("memory", u64), ("device_id", u32), ("ip_version", u32),
                ("xe_cores", u32), ("pcie_gen", i32), ("pcie_width", i32), ("reserved", u32), ("pcie_bytes_per_s", C.c_int64)]


class AbiRow(C.Structure):
    _fields_ = [("name", C.c_char_p), ("offset", u32), ("size", u32)]


class BatchRun(C.Structure):
    _fields_ = [("n", u32), ("pos0", u32), ("slot", u32), ("row0", u32)]


STRUCTS = {"engine_config": Config, "engine_info": Info, "engine_settings": Settings, "engine_page_change": PageChange,
           "engine_prompt_piece": PromptPiece, "engine_step_plan": StepPlan, "engine_event": Event, "engine_timing": Timing,
           "engine_image": Image, "engine_stats": Stats, "engine_slot_stats": SlotStats, "engine_card": Card, "engine_abi_row": AbiRow}

_lib = None


class EngineError(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(f"status {status}: {message}")
        self.status = status


def lib():
    """The loaded library; raises when it has not been built (python -m c0ven_b200.build)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(f"{LIB_PATH} is not built: run `python -m c0ven_b200.build` (there is no other path)")
        L = C.CDLL(LIB_PATH)
        vp = C.c_void_p
        L.engine_open.argtypes = [C.POINTER(Config), C.POINTER(Info), C.POINTER(vp)]
        L.engine_admit.argtypes = [vp, u32, C.POINTER(Settings), C.POINTER(i32), u32]
        L.engine_admit_images.argtypes = [vp, u32, C.POINTER(Image), u32]
        L.engine_release.argtypes = [vp, u32]
        L.engine_submit.argtypes = [vp, C.POINTER(StepPlan)]
        L.engine_poll.argtypes = [vp, C.POINTER(Event), u32, C.POINTER(u32)]
        L.engine_wait.argtypes = [vp, u32]
        L.engine_checkpoint.argtypes = [vp, u32, u32]
        L.engine_restore.argtypes = [vp, u32, u32]
        L.engine_drop.argtypes = [vp, u32]
        L.engine_read_timing.argtypes = [vp, C.POINTER(Timing), u32, C.POINTER(u32)]
        L.engine_read_stats.argtypes = [vp, C.POINTER(Stats)]
        L.engine_read_slot_stats.argtypes = [vp, u32, C.POINTER(SlotStats)]
        L.engine_sleep.argtypes = [vp]
        L.engine_wake.argtypes = [vp, C.POINTER(Info)]
        L.engine_last_error.argtypes = [vp]
        L.engine_last_error.restype = C.c_char_p
        L.engine_close.argtypes = [vp]
        L.engine_close.restype = None
        L.engine_queue_stuck.restype = C.c_int
        L.engine_cards.argtypes = [C.POINTER(Card), u32, C.POINTER(u32)]
        L.engine_abi_layout.argtypes = [C.POINTER(AbiRow), u32]
        L.engine_abi_layout.restype = u32
        L.engine_read_batch.argtypes = [vp, vp, u32, C.POINTER(u32), C.POINTER(BatchRun), u32, C.POINTER(u32)]
        _lib = L
    return _lib


def abi_layout():
    """The library's own table: [(name, offset, size)], fields as "struct.field", then the structs."""
    L = lib()
    n = L.engine_abi_layout(None, 0)
    rows = (AbiRow * n)()
    L.engine_abi_layout(rows, n)
    return [(r.name.decode(), r.offset, r.size) for r in rows]


class Engine:
    """An open engine: admit requests, submit plans, read events (what the reference's NativeEngine does over its core)."""

    def __init__(self, model_path: str, slots: int = 1, max_ctx: int = 0, prompt_chunk: int = 0, checkpoints: int = 0):
        self._h = None
        L = lib()
        cfg = Config(model_path=str(model_path).encode(), slots=slots, max_ctx=max_ctx, prompt_chunk=prompt_chunk, checkpoints=checkpoints)
        self.info = Info()
        h = C.c_void_p()
        st = L.engine_open(C.byref(cfg), C.byref(self.info), C.byref(h))
        if st != OK:
            raise EngineError(st, L.engine_last_error(None).decode())
        self._h = h

    def _check(self, st: int):
        if st != OK:
            raise EngineError(st, lib().engine_last_error(self._h).decode())

    def admit(self, slot: int, prompt, max_tokens: int = 16, stop=(), **settings):
        s = Settings(max_tokens=max_tokens, n_stop=len(stop), penalty_repeat=1.0, **settings)
        for i, t in enumerate(stop):
            s.stop[i] = t
        arr = (i32 * len(prompt))(*prompt)
        self._check(lib().engine_admit(self._h, slot, C.byref(s), arr, len(prompt)))

    def release(self, slot: int):
        self._check(lib().engine_release(self._h, slot))

    def submit(self, decode=(), pieces=(), pages=()):
        """One plan: decode slots, prompt pieces [(slot, tokens)], page changes [(slot, logical, page, source, cells)]."""
        p = StepPlan(nslots=len(decode), npieces=len(pieces), npages=len(pages))
        for i, s in enumerate(decode):
            p.slots[i] = s
        for i, (s, n) in enumerate(pieces):
            p.pieces[i] = PromptPiece(s, n)
        keep = (PageChange * max(len(pages), 1))(*[PageChange(*c) for c in pages])
        p.pages = keep if pages else None
        self._check(lib().engine_submit(self._h, C.byref(p)))

    def poll(self, cap: int = 256):
        buf, n = (Event * cap)(), u32(0)
        self._check(lib().engine_poll(self._h, buf, cap, C.byref(n)))
        return [(e.kind, e.slot, e.token, e.value) for e in buf[:n.value]]

    def wait(self, timeout_ms: int = 1000) -> bool:
        return lib().engine_wait(self._h, timeout_ms) == OK

    def run_until_step(self, seq: int, timeout_s: float = 120.0):
        """Events up to and including plan `seq`'s ENGINE_EVENT_STEP."""
        import time

        out, t0 = [], time.time()
        while time.time() - t0 < timeout_s:
            self.wait(200)
            for ev in self.poll():
                out.append(ev)
                if ev[0] == EVENT_STEP and ev[3] >= seq:
                    return out
        raise TimeoutError(f"plan {seq} did not finish")

    def timing(self, cap: int = 4096):
        buf, n = (Timing * cap)(), u32(0)
        self._check(lib().engine_read_timing(self._h, buf, cap, C.byref(n)))
        return [(t.kind, t.plan, t.rows, t.misses, t.start_ns, t.end_ns) for t in buf[:n.value]]

    def stats(self) -> dict:
        s = Stats()
        self._check(lib().engine_read_stats(self._h, C.byref(s)))
        return {n: getattr(s, n) for n in _STATS}

    def read_batch(self, n_embd: int):
        """The last plan's batch: its hidden rows [rows][n_embd] and its runs [(n, pos0, slot, row0)]."""
        import numpy as np

        rows, nruns = u32(0), u32(0)
        self._check(lib().engine_read_batch(self._h, None, 0, C.byref(rows), None, 0, C.byref(nruns)))
        hidden = np.empty((rows.value, n_embd), dtype=np.float32)
        runs = (BatchRun * max(nruns.value, 1))()
        self._check(lib().engine_read_batch(self._h, hidden.ctypes.data_as(C.c_void_p), rows.value, C.byref(rows), runs, nruns.value, C.byref(nruns)))
        return hidden, [(r.n, r.pos0, r.slot, r.row0) for r in runs[:nruns.value]]

    def checkpoint(self, slot: int, cid: int):
        self._check(lib().engine_checkpoint(self._h, slot, cid))

    def restore(self, slot: int, cid: int):
        self._check(lib().engine_restore(self._h, slot, cid))

    def sleep(self):
        self._check(lib().engine_sleep(self._h))

    def wake(self):
        self._check(lib().engine_wake(self._h, C.byref(self.info)))

    def close(self):
        if self._h is not None:
            lib().engine_close(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
