"""On a B200: a layer made from a GGUF file (moe_layer_create_from_gguf) gives the bits of the same layer made from
raw pointers (moe_layer_create), for whole files and for an expert-parallel slice of one; and still matches the oracle."""
import numpy as np
import pytest

from c0ven_b200 import MoELayer, synth
from c0ven_b200.layer import GgufFile
from oracle import oracle as O

pytestmark = pytest.mark.gpu
pytest.importorskip("gguf")


def _bf16(a):
    u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)
    return (((u + 0x7FFF + ((u >> 16) & 1)) >> 16) << 16).astype(np.uint32).view(np.float32)


def test_layer_from_file_equals_layer_from_pointers(tmp_path):
    layers = [synth.make_layer(n_embd=512, n_ff=256, n_experts=32, n_used=4, gate_type=synth.Q4_K, down_type=synth.Q6_K,
                               shexp_gate_type=synth.Q8_0, shexp_down_type=synth.Q8_0, seed=600 + i) for i in range(2)]
    for L in layers:  # the file stores the router and the gate vector as bf16: the raw-pointer layers get the same values
        L["router"], L["shexp_gate_inp"] = _bf16(L["router"]), _bf16(L["shexp_gate_inp"])
    path = tmp_path / "layers.gguf"
    synth.write_gguf(path, layers, router_type="bf16")
    f = GgufFile(path)
    x = synth.make_input(200, 512, seed=15)
    for i, L in enumerate(layers):
        a = MoELayer.from_gguf(f, i, max_tokens=256)           # n_used from the file's expert_used_count
        b = MoELayer(L, max_tokens=256)
        assert (a.n_embd, a.n_ff, a.n_experts, a.n_used) == (512, 256, 32, 4)
        for T in (3, 200):
            oa, ob = a.forward(x[:T]), b.forward(x[:T])
            assert np.array_equal(oa, ob)
            assert np.array_equal(a.route(T)[0], b.route(T)[0])
            ref = O.moe_forward(L, x[:T])[0]
            assert np.abs(oa - ref).max() / np.abs(ref).max() <= 1e-2
        a.close(), b.close()
    f.close()
