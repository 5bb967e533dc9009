"""moe_route_rows_static, the router that allocates nothing: for callers that have no device memory left to ask for
while a step runs (everything was shared out at load) or that cannot afford the allocator's device-wide wait. Its
scratch is a fixed array inside the library. Checked here through the C ABI against the layer's own router
(moe_layer_forward, then moe_layer_read_route) on two calls in a row, the second with other rows, so that what the
first call left in the shared scratch is seen not to matter. Collected last, so a run that stops at the first failure
has already run every other test."""
import numpy as np
import pytest

from c0ven_b200 import MoELayer, _lib, synth

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
        assert np.allclose(w_dev.cpu().numpy(), w, rtol=1e-5, atol=1e-7)      # the tolerance the parity tests use for w
        logit = (x.astype(np.float64) @ layer["shexp_gate_inp"].astype(np.float64))
        assert np.allclose(gate_dev.cpu().numpy(), 1 / (1 + np.exp(-logit)), rtol=1e-5)
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
