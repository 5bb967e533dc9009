"""ctypes binding of libc0ven_moe.so (include/moe_layer.h). The library is required: nothing here falls back to
another implementation, and a missing library is an ImportError-like failure at first use."""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libc0ven_moe.so")

MOE_OK, MOE_ERROR, MOE_BAD_ARGUMENT, MOE_BUSY, MOE_TIMEOUT = range(5)
FLAG_PROFILE, FLAG_NO_TENSOR, FLAG_GATHER_IN_KERNEL = 1, 2, 4
STAGES = ("quantize", "router", "pack", "gate_up", "down", "shared", "combine", "copies")

SYMBOLS = ("moe_layer_create", "moe_layer_destroy", "moe_layer_forward", "moe_layer_forward_device", "moe_layer_sync",
           "moe_layer_read_route", "moe_layer_read_stats", "moe_layer_stage_ms", "moe_layer_set_profiling", "moe_layer_stream", "moe_last_error",
           "moe_abi_layout", "moe_to_runs", "moe_from_runs",
           "moe_route_rows_static", "moe_route_rows_static_error", "moe_layer_route_device", "moe_layer_read_counts", "moe_layer_counts_device",
           "moe_layer_wire_row_bytes", "moe_layer_received_ids_device", "moe_layer_gather_rows_device", "moe_layer_experts_device", "moe_layer_shared_device",
           "moe_layer_combine_device", "moe_layer_read_groups", "moe_layer_read_quantized", "moe_layer_read_logits",
           "moe_layer_read_config", "moe_layer_forward_residual_device", "moe_rmsnorm_rows_device", "moe_layer_dispatch_row_bytes", "moe_layer_dispatch_plan_device", "moe_layer_dispatch_rows_device",
           "moe_layer_experts_partial_device", "moe_layer_combine_partials_device", "moe_gguf_open", "moe_gguf_close", "moe_gguf_layers", "moe_gguf_tensors", "moe_layer_create_from_gguf")


class Config(C.Structure):
    _fields_ = [("n_embd", C.c_uint32), ("n_ff", C.c_uint32), ("n_experts", C.c_uint32), ("n_used", C.c_uint32),
                ("gate_type", C.c_uint32), ("down_type", C.c_uint32), ("shexp_gate_type", C.c_uint32),
                ("shexp_down_type", C.c_uint32), ("expert_first", C.c_uint32), ("expert_count", C.c_uint32),
                ("max_tokens", C.c_uint32), ("device", C.c_int32), ("swiglu_limit", C.c_float), ("flags", C.c_uint32),
                ("tensor_min_rows", C.c_uint32), ("max_expert_rows", C.c_uint32), ("host_chunk_rows", C.c_uint32)]


class Weights(C.Structure):
    _fields_ = [("router", C.c_void_p), ("shexp_gate_inp", C.c_void_p), ("router_bias", C.c_void_p),
                ("gate_exps", C.c_void_p), ("up_exps", C.c_void_p), ("down_exps", C.c_void_p),
                ("gate_shexp", C.c_void_p), ("up_shexp", C.c_void_p), ("down_shexp", C.c_void_p)]


class Tile(C.Structure):
    _fields_ = [("expert", C.c_uint32), ("slot", C.c_uint32), ("start", C.c_uint32), ("count", C.c_uint32)]


class Group(C.Structure):
    _fields_ = [("slot", C.c_uint32), ("start", C.c_uint32), ("n", C.c_uint32)]


class GgufTensor(C.Structure):
    _fields_ = [("name", C.c_char_p), ("type", C.c_uint32), ("n_dims", C.c_uint32), ("shape", C.c_uint64 * 4),
                ("offset", C.c_uint64), ("bytes", C.c_uint64)]


class Stats(C.Structure):
    _fields_ = [(n, C.c_uint64) for n in ("calls", "rows", "assignments", "kernels", "h2d_bytes", "d2h_bytes",
                                          "last_tiles", "last_experts_hit", "last_tensor_rows")]


class AbiRow(C.Structure):
    _fields_ = [("name", C.c_char_p), ("offset", C.c_uint32), ("size", C.c_uint32)]


STRUCTS = {"moe_gguf_tensor": GgufTensor, "moe_layer_config": Config, "moe_layer_weights": Weights, "moe_tile": Tile, "moe_group": Group, "moe_layer_stats": Stats,
           "moe_abi_row": AbiRow}

_lib = None


class LibraryMissing(RuntimeError):
    pass


def lib():
    """The loaded library. Raises LibraryMissing when it has not been built (python -m c0ven_b200.build)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise LibraryMissing(f"{LIB_PATH} is not built: run `python -m c0ven_b200.build` (there is no other path)")
        L = C.CDLL(LIB_PATH)
        vp, u32 = C.c_void_p, C.c_uint32
        L.moe_layer_create.argtypes = [C.POINTER(Config), C.POINTER(Weights), C.POINTER(vp)]
        L.moe_layer_destroy.argtypes = [vp]
        L.moe_layer_destroy.restype = None
        L.moe_layer_forward.argtypes = [vp, vp, u32, vp]
        L.moe_layer_forward_device.argtypes = [vp, vp, u32, vp, vp]
        L.moe_layer_forward_residual_device.argtypes = [vp, vp, u32, vp, vp, vp]
        L.moe_rmsnorm_rows_device.argtypes = [vp, vp, u32, u32, C.c_float, vp, vp]
        L.moe_layer_sync.argtypes = [vp, u32]
        L.moe_layer_read_route.argtypes = [vp, vp, vp, vp, vp, u32, C.POINTER(u32)]
        L.moe_layer_read_stats.argtypes = [vp, C.POINTER(Stats)]
        L.moe_layer_read_groups.argtypes = [vp, vp, u32, C.POINTER(u32)]
        L.moe_layer_read_quantized.argtypes = [vp, u32, vp, vp, vp, C.POINTER(u32)]
        L.moe_layer_read_config.argtypes = [vp, C.POINTER(Config)]
        L.moe_layer_dispatch_row_bytes.argtypes = [vp]
        L.moe_layer_dispatch_row_bytes.restype = u32
        L.moe_layer_dispatch_plan_device.argtypes = [vp, vp, vp]
        L.moe_layer_dispatch_rows_device.argtypes = [vp, vp, vp]
        L.moe_layer_experts_partial_device.argtypes = [vp, vp, u32, u32, vp, vp]
        L.moe_layer_combine_partials_device.argtypes = [vp, vp, vp, vp]
        L.moe_gguf_open.argtypes = [C.c_char_p, C.POINTER(vp)]
        L.moe_gguf_close.argtypes = [vp]
        L.moe_gguf_close.restype = None
        L.moe_gguf_layers.argtypes = [vp]
        L.moe_gguf_layers.restype = u32
        L.moe_gguf_tensors.argtypes = [vp, C.POINTER(GgufTensor), u32]
        L.moe_gguf_tensors.restype = u32
        L.moe_layer_create_from_gguf.argtypes = [vp, u32, C.POINTER(Config), C.POINTER(vp)]
        L.moe_layer_read_logits.argtypes = [vp, vp, C.POINTER(u32), C.POINTER(C.c_float), C.POINTER(C.c_float)]
        L.moe_layer_stage_ms.argtypes = [vp, vp]
        L.moe_layer_set_profiling.argtypes = [vp, u32]
        L.moe_layer_stream.argtypes = [vp]
        L.moe_layer_stream.restype = vp
        L.moe_last_error.argtypes = [vp]
        L.moe_last_error.restype = C.c_char_p
        L.moe_to_runs.argtypes = [u32, vp, C.c_uint64, vp]
        L.moe_from_runs.argtypes = [u32, vp, C.c_uint64, vp]
        L.moe_layer_route_device.argtypes = [vp, vp, u32, vp]
        L.moe_layer_read_counts.argtypes = [vp, vp, vp]
        L.moe_layer_counts_device.argtypes = [vp, vp, vp]
        L.moe_layer_received_ids_device.argtypes = [vp, vp, u32, vp, vp]
        L.moe_layer_wire_row_bytes.argtypes = [vp]
        L.moe_layer_wire_row_bytes.restype = u32
        L.moe_layer_gather_rows_device.argtypes = [vp, vp, vp, vp]
        L.moe_layer_experts_device.argtypes = [vp, vp, vp, u32, vp, u32, vp]
        L.moe_layer_shared_device.argtypes = [vp, vp]
        L.moe_layer_combine_device.argtypes = [vp, vp, u32, vp, vp]
        L.moe_route_rows_static.argtypes = [vp, u32, u32, vp, vp, u32, u32, vp, vp, vp, vp]
        L.moe_route_rows_static_error.restype = C.c_char_p
        L.moe_abi_layout.argtypes = [C.POINTER(AbiRow), u32]
        L.moe_abi_layout.restype = u32
        _lib = L
    return _lib


def abi_layout():
    """The library's own table of struct fields: [(name, offset, size)]."""
    L = lib()
    n = L.moe_abi_layout(None, 0)
    rows = (AbiRow * n)()
    L.moe_abi_layout(rows, n)
    return [(r.name.decode(), r.offset, r.size) for r in rows]
