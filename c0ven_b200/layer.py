"""The host side of the MoE layer: the calls the reference's model program makes for a layer's MoE block
(core/models/qwen4exp/model.cpp:1348-1418, prompt.cpp:606-656) and its CPU path's interface
(CpuExperts::compute_many, core/cpu/experts.h:32-53), over the C ABI of include/moe_layer.h."""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import _lib


class MoEError(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(f"status {status}: {message}")
        self.status = status


def _ptr(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def rmsnorm_rows_device(x_ptr: int, weight_ptr: int | None, T: int, n_embd: int, eps: float, out_ptr: int, stream: int | None = None):
    """out[t] = x[t] / sqrt(mean(x[t]^2) + eps) * weight on device rows (addresses), queued on stream."""
    st = _lib.lib().moe_rmsnorm_rows_device(x_ptr, weight_ptr, T, n_embd, eps, out_ptr, stream)
    if st != _lib.MOE_OK:
        raise MoEError(st, "moe_rmsnorm_rows_device refused its arguments or could not launch")


class GgufFile:
    """A GGUF file's tensor table, through the library's reader (moe_gguf_*)."""

    def __init__(self, path: str):
        self._h = None
        h = C.c_void_p()
        st = _lib.lib().moe_gguf_open(str(path).encode(), C.byref(h))
        if st != _lib.MOE_OK:
            raise MoEError(st, _lib.lib().moe_last_error(None).decode())
        self._h = h

    @property
    def layers(self) -> int:
        return _lib.lib().moe_gguf_layers(self._h)

    def tensors(self) -> dict:
        """name -> (ggml type, shape in ggml order, offset in the file, bytes)."""
        L = _lib.lib()
        n = L.moe_gguf_tensors(self._h, None, 0)
        rows = (_lib.GgufTensor * n)()
        L.moe_gguf_tensors(self._h, rows, n)
        return {r.name.decode(): (r.type, tuple(r.shape[:r.n_dims]), r.offset, r.bytes) for r in rows}

    def close(self):
        if self._h is not None:
            _lib.lib().moe_gguf_close(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class MoELayer:
    """One layer's router, experts and shared expert on one GPU.

    layer: a dict with n_embd, n_ff, n_experts, n_used, the four types, router [NE][E] f32, shexp_gate_inp [E] f32,
    optional router_bias [NE] f32, and the experts' matrices as uint8 arrays in the GGUF file's block layout
    (gate_exps, up_exps [NE][F][row bytes], down_exps [NE][E][row bytes], gate_shexp, up_shexp, down_shexp) — what
    c0ven_b200.synth.make_layer returns.
    """

    def __init__(self, layer: dict, max_tokens: int = 4352, device: int = 0, profile: bool = False,
                 expert_first: int = 0, expert_count: int = 0, no_tensor: bool = False, tensor_min_rows: int = 0,
                 max_expert_rows: int = 0, host_chunk_rows: int = 0, own_experts=None, gather_in_kernel: bool = False):
        """own_experts: this GPU's experts' (gate, up, down) arrays, [expert_count][rows][row bytes] each, when they are
        not the slice [expert_first, expert_first + expert_count) of the layer's own arrays."""
        self._h = None
        L = _lib.lib()
        self.n_embd, self.n_ff = layer["n_embd"], layer["n_ff"]
        self.n_experts, self.n_used = layer["n_experts"], layer["n_used"]
        self.max_tokens = max_tokens
        count = expert_count or self.n_experts - expert_first
        has_shared = layer.get("gate_shexp") is not None
        cfg = _lib.Config(self.n_embd, self.n_ff, self.n_experts, self.n_used, layer["gate_type"], layer["down_type"],
                          layer["shexp_gate_type"] if has_shared else 0, layer["shexp_down_type"] if has_shared else 0,
                          expert_first, count, max_tokens, device, float(layer.get("swiglu_limit", 0.0)),
                          (_lib.FLAG_PROFILE if profile else 0) | (_lib.FLAG_NO_TENSOR if no_tensor else 0)
                          | (_lib.FLAG_GATHER_IN_KERNEL if gather_in_kernel else 0), tensor_min_rows, max_expert_rows, host_chunk_rows)
        sl = slice(expert_first, expert_first + count)
        ge, ue, de = own_experts if own_experts is not None else (layer["gate_exps"][sl], layer["up_exps"][sl], layer["down_exps"][sl])
        if len(ge) != count or len(ue) != count or len(de) != count:
            # Refused here as the library refuses a bad shape: it would read past the arrays' ends.
            raise MoEError(_lib.MOE_BAD_ARGUMENT, "the experts' arrays must hold expert_count experts")
        keep = [np.ascontiguousarray(layer["router"], dtype=np.float32),
                np.ascontiguousarray(layer["shexp_gate_inp"], dtype=np.float32) if has_shared else None,
                np.ascontiguousarray(layer["router_bias"], dtype=np.float32) if layer.get("router_bias") is not None else None,
                np.ascontiguousarray(ge), np.ascontiguousarray(ue), np.ascontiguousarray(de),
                np.ascontiguousarray(layer["gate_shexp"]) if has_shared else None,
                np.ascontiguousarray(layer["up_shexp"]) if has_shared else None,
                np.ascontiguousarray(layer["down_shexp"]) if has_shared else None]
        w = _lib.Weights(*[a.ctypes.data if a is not None else None for a in keep])
        h = C.c_void_p()
        st = L.moe_layer_create(C.byref(cfg), C.byref(w), C.byref(h))
        if st != _lib.MOE_OK:
            raise MoEError(st, L.moe_last_error(None).decode())
        self._h = h

    @classmethod
    def from_gguf(cls, gguf: GgufFile, layer: int, n_used: int = 0, max_tokens: int = 4352, device: int = 0, profile: bool = False,
                  expert_first: int = 0, expert_count: int = 0, no_tensor: bool = False, tensor_min_rows: int = 0,
                  max_expert_rows: int = 0, host_chunk_rows: int = 0, swiglu_limit: float = 0.0):
        """Layer `layer` of an open GGUF file: sizes and types come from its tensors (moe_layer_create_from_gguf)."""
        L = _lib.lib()
        cfg = _lib.Config(0, 0, 0, n_used, 0, 0, 0, 0, expert_first, expert_count, max_tokens, device, float(swiglu_limit),
                          (_lib.FLAG_PROFILE if profile else 0) | (_lib.FLAG_NO_TENSOR if no_tensor else 0), tensor_min_rows,
                          max_expert_rows, host_chunk_rows)
        h = C.c_void_p()
        st = L.moe_layer_create_from_gguf(gguf._h, layer, C.byref(cfg), C.byref(h))
        if st != _lib.MOE_OK:
            raise MoEError(st, L.moe_last_error(None).decode())
        self = cls.__new__(cls)
        self._h = h
        got = _lib.Config()
        L.moe_layer_read_config(h, C.byref(got))
        self.n_embd, self.n_ff, self.n_experts, self.n_used = got.n_embd, got.n_ff, got.n_experts, got.n_used
        self.max_tokens = got.max_tokens
        return self

    def _check(self, st: int):
        if st != _lib.MOE_OK:
            raise MoEError(st, _lib.lib().moe_last_error(self._h).decode())

    def close(self):
        if self._h is not None:
            _lib.lib().moe_layer_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def forward(self, x: np.ndarray, out: np.ndarray | None = None) -> np.ndarray:
        """The block on host rows x [T][E] f32; copies in, computes, copies out, waits."""
        x = np.ascontiguousarray(x, dtype=np.float32)
        if x.ndim != 2 or x.shape[1] != self.n_embd:
            raise ValueError("x must be [T][n_embd]")
        if out is None:
            out = np.empty_like(x)
        self._check(_lib.lib().moe_layer_forward(self._h, _ptr(x), x.shape[0], _ptr(out)))
        return out

    def forward_device(self, x_ptr: int, T: int, out_ptr: int, stream: int | None = None):
        """The block on device buffers (addresses), queued without waiting."""
        self._check(_lib.lib().moe_layer_forward_device(self._h, x_ptr, T, out_ptr, stream))

    def forward_residual_device(self, x_ptr: int, T: int, residual_ptr: int, out_ptr: int, stream: int | None = None):
        """out = residual + block(x) on device buffers (addresses), queued without waiting."""
        self._check(_lib.lib().moe_layer_forward_residual_device(self._h, x_ptr, T, residual_ptr, out_ptr, stream))

    def sync(self, timeout_ms: int = 0):
        self._check(_lib.lib().moe_layer_sync(self._h, timeout_ms))

    def route(self, T: int):
        """The last call's ids [T][K], w [T][K], inv [T*K] and tiles [n][4] (expert, slot, start, count)."""
        K = self.n_used
        ids = np.empty((T, K), dtype=np.int32)
        w = np.empty((T, K), dtype=np.float32)
        inv = np.empty(T * K, dtype=np.uint32)
        cap = T * K // 64 + self.n_experts + 1
        tiles = np.empty((cap, 4), dtype=np.uint32)
        n = C.c_uint32(0)
        self._check(_lib.lib().moe_layer_read_route(self._h, _ptr(ids), _ptr(w), _ptr(inv), _ptr(tiles), cap, C.byref(n)))
        return ids, w, inv, tiles[:n.value].copy()

    def groups(self) -> np.ndarray:
        """The last call's groups for the integer-dot kernels, [n][3] (slot, start, n), in expert order."""
        n = C.c_uint32(0)
        self._check(_lib.lib().moe_layer_read_groups(self._h, None, 0, C.byref(n)))
        g = np.empty((max(n.value, 1), 3), dtype=np.uint32)
        self._check(_lib.lib().moe_layer_read_groups(self._h, _ptr(g), n.value, C.byref(n)))
        return g[:n.value].copy()

    def quantized(self, T: int, inner: bool = False):
        """The last call's quantised rows: codes [rows][K] int8, scales [rows][K/32 or K/256] f32, and for q8_K the
        int16 sums [rows][K/16] (else None). inner: the routed experts' h rows in expert order instead of x."""
        rows, Kv = (T * self.n_used, self.n_ff) if inner else (T, self.n_embd)
        k = C.c_uint32(0)
        self._check(_lib.lib().moe_layer_read_quantized(self._h, int(inner), None, None, None, C.byref(k)))
        q = np.empty((rows, Kv), dtype=np.int8)
        d = np.empty((rows, Kv // (256 if k.value else 32)), dtype=np.float32)
        bs = np.empty((rows, Kv // 16), dtype=np.int16) if k.value else None
        self._check(_lib.lib().moe_layer_read_quantized(self._h, int(inner), _ptr(q), _ptr(d), _ptr(bs), C.byref(k)))
        return q, d, bs

    def logits(self, T: int):
        """The last call's router logits [T][n_experts] without the bias, whether they are the tensor-core product's
        approximate ones, and the bound on their error: eps_rel * |x_t| + eps_abs."""
        lg = np.empty((T, self.n_experts), dtype=np.float32)
        ap, er, ea = C.c_uint32(0), C.c_float(0), C.c_float(0)
        self._check(_lib.lib().moe_layer_read_logits(self._h, _ptr(lg), C.byref(ap), C.byref(er), C.byref(ea)))
        return lg, bool(ap.value), er.value, ea.value

    # Expert parallel, stage by stage (device addresses; queued on `stream`, the layer's own when None).
    def route_device(self, x_ptr: int, T: int, stream=None):
        self._check(_lib.lib().moe_layer_route_device(self._h, x_ptr, T, stream))

    def read_counts(self, stream=None) -> np.ndarray:
        cnt = np.empty(self.n_experts, dtype=np.uint32)
        self._check(_lib.lib().moe_layer_read_counts(self._h, _ptr(cnt), stream))
        return cnt

    def counts_device(self, cnt_ptr: int, stream=None):
        self._check(_lib.lib().moe_layer_counts_device(self._h, cnt_ptr, stream))

    def received_ids_device(self, cnt_all_ptr: int, world: int, ids_ptr: int, stream=None):
        self._check(_lib.lib().moe_layer_received_ids_device(self._h, cnt_all_ptr, world, ids_ptr, stream))

    @property
    def wire_row_bytes(self) -> int:
        return _lib.lib().moe_layer_wire_row_bytes(self._h)

    def gather_rows_device(self, rows_ptr: int, ids_ptr: int, stream=None):
        self._check(_lib.lib().moe_layer_gather_rows_device(self._h, rows_ptr, ids_ptr, stream))

    def experts_device(self, rows_ptr: int, ids_ptr: int, R: int, y_ptr: int, y_f16: bool, stream=None):
        self._check(_lib.lib().moe_layer_experts_device(self._h, rows_ptr, ids_ptr, R, y_ptr, int(y_f16), stream))

    def shared_device(self, stream=None):
        self._check(_lib.lib().moe_layer_shared_device(self._h, stream))

    def combine_device(self, y_ptr: int, y_f16: bool, out_ptr: int, stream=None):
        self._check(_lib.lib().moe_layer_combine_device(self._h, y_ptr, int(y_f16), out_ptr, stream))

    # Expert parallel with one row per (token, GPU).
    @property
    def dispatch_row_bytes(self) -> int:
        return _lib.lib().moe_layer_dispatch_row_bytes(self._h)

    def dispatch_plan_device(self, totals_ptr: int, stream=None):
        self._check(_lib.lib().moe_layer_dispatch_plan_device(self._h, totals_ptr, stream))

    def dispatch_rows_device(self, rows_ptr: int, stream=None):
        self._check(_lib.lib().moe_layer_dispatch_rows_device(self._h, rows_ptr, stream))

    def experts_partial_device(self, rows_ptr: int, R: int, assignments: int, y_ptr: int, stream=None):
        self._check(_lib.lib().moe_layer_experts_partial_device(self._h, rows_ptr, R, assignments, y_ptr, stream))

    def combine_partials_device(self, back_ptr: int, out_ptr: int, stream=None):
        self._check(_lib.lib().moe_layer_combine_partials_device(self._h, back_ptr, out_ptr, stream))

    def stats(self) -> dict:
        s = _lib.Stats()
        self._check(_lib.lib().moe_layer_read_stats(self._h, C.byref(s)))
        return {n: getattr(s, n) for n, _ in _lib.Stats._fields_}

    def set_profiling(self, on: bool):
        self._check(_lib.lib().moe_layer_set_profiling(self._h, int(on)))

    def stage_ms(self) -> dict:
        ms = np.zeros(len(_lib.STAGES), dtype=np.float32)
        self._check(_lib.lib().moe_layer_stage_ms(self._h, _ptr(ms)))
        return dict(zip(_lib.STAGES, ms.tolist()))

    @property
    def stream(self) -> int:
        return _lib.lib().moe_layer_stream(self._h)
