"""ctypes binding of the CPU oracle (oracle/moe_oracle.c).

Test infrastructure only: tests, the smoke check and the bench's CPU-baseline leg import this. The product path never
does. Each function is the C function of the same name; moe_oracle.h cites the reference lines they restate.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "libmoe_oracle.so")

Q8_0, Q4_K, Q6_K, Q8_K, IQ3_XXS, IQ4_NL, IQ3_S, IQ2_S, IQ4_XS, Q2_0 = 8, 12, 14, 15, 18, 20, 21, 22, 23, 42


def build() -> str:
    """Compiles the oracle where its sources are newer than the library (needs gcc and gguf-py)."""
    srcs = [os.path.join(_HERE, f) for f in ("moe_oracle.c", "moe_oracle.h", "Makefile")]
    if not os.path.exists(_SO) or any(os.path.getmtime(s) > os.path.getmtime(_SO) for s in srcs):
        subprocess.run(["make", "-C", _HERE], check=True, capture_output=True)
    return _SO


def build_ref(reference_root: str) -> str | None:
    """Compiles the reference's shared layout headers, where they lie under reference_root, into oracle/_ref/
    (ref_layout.cpp); None when that tree is not there."""
    if not os.path.exists(os.path.join(reference_root, "shared", "quant.h")):
        return None
    subprocess.run(["make", "-C", _HERE, "REFERENCE=" + os.path.abspath(reference_root), "ref"], check=True, capture_output=True)
    return os.path.join(_HERE, "_ref", "libref_layout.so")


class Tile(C.Structure):
    _fields_ = [("expert", C.c_uint32), ("slot", C.c_uint32), ("start", C.c_uint32), ("count", C.c_uint32)]


class _Shape(C.Structure):
    _fields_ = [("gate_type", C.c_uint32), ("down_type", C.c_uint32), ("n_embd", C.c_uint32), ("n_ff", C.c_uint32),
                ("swiglu_limit", C.c_float)]


class _Job(C.Structure):
    _fields_ = [("gate", C.c_void_p), ("up", C.c_void_p), ("down", C.c_void_p), ("tok", C.c_uint32), ("w", C.c_float)]


class _Layer(C.Structure):
    _fields_ = [("n_embd", C.c_uint32), ("n_ff", C.c_uint32), ("n_experts", C.c_uint32), ("n_used", C.c_uint32),
                ("gate_type", C.c_uint32), ("down_type", C.c_uint32), ("shexp_gate_type", C.c_uint32),
                ("shexp_down_type", C.c_uint32), ("swiglu_limit", C.c_float),
                ("router", C.c_void_p), ("shexp_gate_inp", C.c_void_p), ("router_bias", C.c_void_p),
                ("gate_exps", C.c_void_p), ("up_exps", C.c_void_p), ("down_exps", C.c_void_p),
                ("gate_shexp", C.c_void_p), ("up_shexp", C.c_void_p), ("down_shexp", C.c_void_p)]


_lib = None


def lib():
    global _lib
    if _lib is None:
        build()
        L = C.CDLL(_SO)
        L.orc_block_values.restype = C.c_uint32
        L.orc_block_bytes.restype = C.c_uint32
        L.orc_vec_dot_type.restype = C.c_uint32
        L.orc_row_bytes.restype = C.c_uint64
        L.orc_row_bytes.argtypes = [C.c_uint32, C.c_uint64]
        L.orc_dequantize_row.argtypes = [C.c_uint32, C.c_void_p, C.c_void_p, C.c_int64]
        L.orc_quantize_row.argtypes = [C.c_uint32, C.c_void_p, C.c_void_p, C.c_int64]
        L.orc_vec_dot.restype = C.c_float
        L.orc_vec_dot.argtypes = [C.c_uint32, C.c_int64, C.c_void_p, C.c_void_p]
        L.orc_to_runs.argtypes = [C.c_uint32, C.c_void_p, C.c_uint64, C.c_void_p]
        L.orc_from_runs.argtypes = [C.c_uint32, C.c_void_p, C.c_uint64, C.c_void_p]
        L.orc_router_logits.argtypes = [C.c_void_p, C.c_uint32, C.c_uint32, C.c_void_p, C.c_void_p, C.c_void_p,
                                        C.c_uint32, C.c_void_p]
        L.orc_router_topk.argtypes = [C.c_void_p, C.c_uint32, C.c_uint32, C.c_uint32, C.c_void_p, C.c_void_p,
                                      C.c_void_p]
        L.orc_pack.restype = C.c_uint32
        L.orc_pack.argtypes = [C.c_void_p, C.c_uint32, C.c_uint32, C.c_uint32, C.c_void_p, C.c_void_p, C.c_void_p,
                               C.c_void_p]
        L.orc_compute_many.argtypes = [C.c_void_p, C.c_void_p, C.c_uint32, C.c_uint32, C.c_void_p, C.c_uint64,
                                       C.c_void_p, C.c_uint64, C.c_int]
        L.orc_moe_forward.argtypes = [C.c_void_p, C.c_void_p, C.c_uint32, C.c_void_p, C.c_void_p, C.c_void_p,
                                      C.c_void_p, C.c_void_p, C.c_void_p, C.c_int]
        L.orc_threads.restype = C.c_int
        L.orc_set_threads.argtypes = [C.c_int]
        L.orc_set_threads.restype = None
        _lib = L
    return _lib


def _p(a):
    return a.ctypes.data_as(C.c_void_p) if a is not None else None


def block_values(t): return lib().orc_block_values(t)
def block_bytes(t): return lib().orc_block_bytes(t)
def vec_dot_type(t): return lib().orc_vec_dot_type(t)
def row_bytes(t, n): return lib().orc_row_bytes(t, n)
def threads(): return lib().orc_threads()


def host_threads() -> int:
    """The cores this process may run on (the reference's rule for sizing its pool, docs/DESIGN.md:694-696), set as
    the oracle's thread count whatever OMP_NUM_THREADS says (launchers such as torchrun set it to 1)."""
    n = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    lib().orc_set_threads(n)
    return n


def dequantize(t: int, blocks: np.ndarray, n: int) -> np.ndarray:
    blocks = np.ascontiguousarray(blocks, dtype=np.uint8)
    y = np.empty(n, dtype=np.float32)
    lib().orc_dequantize_row(t, _p(blocks), _p(y), n)
    return y


def quantize(act_type: int, x: np.ndarray) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float32)
    y = np.zeros(row_bytes(act_type, x.size), dtype=np.uint8)
    lib().orc_quantize_row(act_type, _p(x), _p(y), x.size)
    return y


def vec_dot(t: int, w: np.ndarray, a: np.ndarray, n: int) -> float:
    return float(lib().orc_vec_dot(t, n, _p(np.ascontiguousarray(w)), _p(np.ascontiguousarray(a))))


def to_runs(t: int, blocks: np.ndarray) -> np.ndarray:
    blocks = np.ascontiguousarray(blocks, dtype=np.uint8)
    out = np.empty_like(blocks)
    lib().orc_to_runs(t, _p(blocks), blocks.size // block_bytes(t), _p(out))
    return out


def from_runs(t: int, runs: np.ndarray) -> np.ndarray:
    runs = np.ascontiguousarray(runs, dtype=np.uint8)
    out = np.empty_like(runs)
    lib().orc_from_runs(t, _p(runs), runs.size // block_bytes(t), _p(out))
    return out


def router_logits(x, W, wsg, bias=None):
    x = np.ascontiguousarray(x, dtype=np.float32)
    W = np.ascontiguousarray(W, dtype=np.float32)
    wsg = np.ascontiguousarray(wsg, dtype=np.float32)
    T, E = x.shape
    NE = W.shape[0]
    rl = np.empty((T, NE + 1), dtype=np.float32)
    bias = None if bias is None else np.ascontiguousarray(bias, dtype=np.float32)
    lib().orc_router_logits(_p(x), T, E, _p(W), _p(wsg), _p(bias), NE, _p(rl))
    return rl


def router_topk(rl, K):
    rl = np.ascontiguousarray(rl, dtype=np.float32)
    T, N = rl.shape
    ids = np.empty((T, K), dtype=np.int32)
    w = np.empty((T, K), dtype=np.float32)
    gs = np.empty(T, dtype=np.float32)
    lib().orc_router_topk(_p(rl), T, N - 1, K, _p(ids), _p(w), _p(gs))
    return ids, w, gs


def pack(ids, NE, first_expert=0):
    ids = np.ascontiguousarray(ids, dtype=np.int32).reshape(-1)
    A = ids.size
    cnt = np.empty(NE, dtype=np.uint32)
    base = np.empty(NE, dtype=np.uint32)
    inv = np.empty(A, dtype=np.uint32)
    tiles = (Tile * (A // 64 + NE + 1))()
    nt = lib().orc_pack(_p(ids), A, NE, first_expert, _p(cnt), _p(base), _p(inv), tiles)
    t = np.array([(x.expert, x.slot, x.start, x.count) for x in tiles[:nt]], dtype=np.uint32).reshape(nt, 4)
    return cnt, base, inv, t


def compute_many(gate_type, down_type, E, F, jobs, x, swiglu_limit=0.0, nthreads=0):
    """jobs: list of (gate, up, down, tok, w) with the three matrices as uint8 arrays in the file's layout."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    ntok = x.shape[0]
    arr = (_Job * len(jobs))()
    keep = []
    for i, (g, u, d, tok, w) in enumerate(jobs):
        keep += [g, u, d]
        arr[i] = _Job(g.ctypes.data, u.ctypes.data, d.ctypes.data, tok, w)
    y = np.empty((ntok, E), dtype=np.float32)
    shape = _Shape(gate_type, down_type, E, F, swiglu_limit)
    lib().orc_compute_many(C.byref(shape), arr, len(jobs), ntok, _p(x), E, _p(y), E, nthreads)
    return y


def moe_forward(layer: dict, x: np.ndarray, nthreads: int = 0, want_pack: bool = True):
    """layer: the dict c0ven_b200.synth.make_layer returns. Returns out, ids, w, inv, tiles."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    T, E = x.shape
    K, NE = layer["n_used"], layer["n_experts"]
    st = _Layer(E, layer["n_ff"], NE, K, layer["gate_type"], layer["down_type"], layer["shexp_gate_type"],
                layer["shexp_down_type"], layer.get("swiglu_limit", 0.0),
                layer["router"].ctypes.data, layer["shexp_gate_inp"].ctypes.data,
                layer["router_bias"].ctypes.data if layer.get("router_bias") is not None else None,
                layer["gate_exps"].ctypes.data, layer["up_exps"].ctypes.data, layer["down_exps"].ctypes.data,
                layer["gate_shexp"].ctypes.data, layer["up_shexp"].ctypes.data, layer["down_shexp"].ctypes.data)
    out = np.empty((T, E), dtype=np.float32)
    ids = np.empty((T, K), dtype=np.int32)
    w = np.empty((T, K), dtype=np.float32)
    inv = np.empty(T * K, dtype=np.uint32) if want_pack else None
    tiles = (Tile * (T * K // 64 + NE + 1))() if want_pack else None
    nt = C.c_uint32(0)
    lib().orc_moe_forward(C.byref(st), _p(x), T, _p(out), _p(ids), _p(w), _p(inv), tiles, C.byref(nt), nthreads)
    tl = None
    if want_pack:
        tl = np.array([(t.expert, t.slot, t.start, t.count) for t in tiles[:nt.value]], dtype=np.uint32).reshape(-1, 4)
    return out, ids, w, inv, tl
