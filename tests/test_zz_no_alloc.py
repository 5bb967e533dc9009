"""moe_route_rows_static, the router that allocates nothing: for callers that have no device memory left to ask for
while a step runs (everything was shared out at load) or that cannot afford the allocator's device-wide wait. Its
scratch is a fixed array inside the library. Checked here through the C ABI against the layer's own router
(moe_layer_forward, then moe_layer_read_route) on two calls in a row, the second with other rows, so that what the
first call left in the shared scratch is seen not to matter. Collected last, so a run that stops at the first failure
has already run every other test."""
import numpy as np
import pytest

from c0ven_b200 import MoELayer, _lib, synth
from oracle import oracle as O

pytestmark = pytest.mark.gpu


def test_static_router_matches_the_layers_router_twice():
    import torch

    E, NE, K = 512, 64, 6
    layer = synth.make_layer(n_embd=E, n_ff=256, n_experts=NE, n_used=K, gate_type=synth.Q8_0, zipf_s=1.1, seed=77)
    gpu = MoELayer(layer, max_tokens=64, device=0)
    L = _lib.lib()
    torch.cuda.set_device(0)
    rows = np.concatenate([layer["router"], layer["shexp_gate_inp"][None]], 0)
    router_dev = torch.from_numpy(rows).cuda()
    bias_dev = torch.from_numpy(layer["router_bias"]).cuda()
    for call, T in enumerate((64, 23)):  # the second call is shorter: stale rows stay behind it in the scratch
        x = synth.make_input(T, E, seed=300 + call)
        gpu.forward(x)
        ids, w, _, _ = gpu.route(T)
        x_dev = torch.from_numpy(x).cuda()
        ids_dev = torch.full((T, K), -1, dtype=torch.int32, device="cuda")
        w_dev = torch.full((T, K), float("nan"), device="cuda")
        gate_dev = torch.full((T,), float("nan"), device="cuda")
        torch.cuda.synchronize()
        st = L.moe_route_rows_static(x_dev.data_ptr(), T, E, router_dev.data_ptr(), bias_dev.data_ptr(), NE, K,
                                     ids_dev.data_ptr(), w_dev.data_ptr(), gate_dev.data_ptr(), None)
        assert st == _lib.MOE_OK, L.moe_route_rows_static_error()
        torch.cuda.synchronize()
        assert np.array_equal(ids_dev.cpu().numpy(), ids)                     # expert ids: bit for bit
        rids, rw, rgs = O.router_topk(O.router_logits(x, layer["router"], layer["shexp_gate_inp"], layer["router_bias"]), K)
        assert np.array_equal(ids_dev.cpu().numpy(), rids)                    # and against the CPU oracle, not only CUDA against CUDA
        assert np.allclose(w_dev.cpu().numpy(), rw, rtol=1e-5, atol=1e-7)
        assert np.allclose(gate_dev.cpu().numpy(), rgs, rtol=1e-5)
        assert np.allclose(w_dev.cpu().numpy(), w, rtol=1e-5, atol=1e-7)      # the tolerance the parity tests use for w
        logit = (x.astype(np.float64) @ layer["shexp_gate_inp"].astype(np.float64))
        assert np.allclose(gate_dev.cpu().numpy(), 1 / (1 + np.exp(-logit)), rtol=1e-5)
    gpu.close()


def _static_route(x, rows, bias, NE, K):
    import torch

    L = _lib.lib()
    T, E = x.shape
    x_dev, router_dev = torch.from_numpy(x).cuda(), torch.from_numpy(rows).cuda()
    bias_dev = torch.from_numpy(bias).cuda() if bias is not None else None
    ids_dev = torch.full((T, K), -1, dtype=torch.int32, device="cuda")
    w_dev = torch.full((T, K), float("nan"), device="cuda")
    gate_dev = torch.full((T,), float("nan"), device="cuda")
    torch.cuda.synchronize()
    st = L.moe_route_rows_static(x_dev.data_ptr(), T, E, router_dev.data_ptr(), bias_dev.data_ptr() if bias is not None else None, NE, K,
                                 ids_dev.data_ptr(), w_dev.data_ptr(), gate_dev.data_ptr(), None)
    assert st == _lib.MOE_OK, L.moe_route_rows_static_error()
    torch.cuda.synchronize()
    return ids_dev.cpu().numpy(), w_dev.cpu().numpy(), gate_dev.cpu().numpy()


def test_static_router_at_its_limits_and_at_the_benchmark_shape():
    """The largest sizes the entry point takes (64 rows, then 33 so that the second chunk is ragged; hidden 4096, which
    needs the opt-in to 132 KB of shared memory its set-up makes; 512 experts; top 16; no bias), against the CPU oracle;
    then the benchmark's shape (hidden 2048, 512 experts, top 10, Zipf bias) against the oracle and the layer's router."""
    import torch

    torch.cuda.set_device(0)
    rng = np.random.default_rng(5)
    E, NE, K = 4096, 512, 16
    W = (rng.standard_normal((NE, E)) * 0.02).astype(np.float32)
    g = (rng.standard_normal(E) * 0.02).astype(np.float32)
    rows = np.concatenate([W, g[None]], 0)
    for T in (64, 33):
        x = synth.make_input(T, E, seed=400 + T)
        ids, w, gate = _static_route(x, rows, None, NE, K)
        rids, rw, rgs = O.router_topk(O.router_logits(x, W, g, None), K)
        assert np.array_equal(ids, rids)
        assert np.allclose(w, rw, rtol=1e-5, atol=1e-7) and np.allclose(gate, rgs, rtol=1e-5)
    layer = synth.make_layer(gate_type=synth.Q8_0, zipf_s=1.1, seed=78)
    gpu = MoELayer(layer, max_tokens=64, device=0, no_tensor=True)
    x = synth.make_input(48, 2048, seed=500)
    gpu.forward(x)
    lids, lw, _, _ = gpu.route(48)
    rows = np.concatenate([layer["router"], layer["shexp_gate_inp"][None]], 0)
    ids, w, gate = _static_route(x, rows, layer["router_bias"], 512, 10)
    rids, rw, rgs = O.router_topk(O.router_logits(x, layer["router"], layer["shexp_gate_inp"], layer["router_bias"]), 10)
    assert np.array_equal(ids, rids) and np.array_equal(ids, lids)
    assert np.allclose(w, rw, rtol=1e-5, atol=1e-7) and np.allclose(w, lw, rtol=1e-5, atol=1e-7) and np.allclose(gate, rgs, rtol=1e-5)
    gpu.close()


def test_static_router_refuses_what_its_scratch_cannot_hold():
    import torch

    L = _lib.lib()
    torch.cuda.set_device(0)
    buf = torch.zeros(1024, device="cuda")
    p = buf.data_ptr()
    assert L.moe_route_rows_static(p, 65, 512, p, None, 64, 4, p, p, p, None) == _lib.MOE_BAD_ARGUMENT
    assert b"64" in L.moe_route_rows_static_error()
    assert L.moe_route_rows_static(p, 8, 512, p, None, 544, 4, p, p, p, None) == _lib.MOE_BAD_ARGUMENT
    assert L.moe_route_rows_static(p, 0, 512, p, None, 64, 4, p, p, p, None) == _lib.MOE_BAD_ARGUMENT
    assert L.moe_route_rows_static(p + 4, 8, 512, p, None, 64, 4, p, p, p, None) == _lib.MOE_BAD_ARGUMENT  # x not 16-byte aligned
    assert b"aligned" in L.moe_route_rows_static_error()
