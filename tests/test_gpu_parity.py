"""On a B200: the CUDA layer, through the C ABI, against the CPU oracle on the same seeded inputs. Expert ids, the
pack permutation and the tiles are compared bit for bit; outputs by the reference's error measure,
max|a - b| / max|b| (docs/TESTING.md:47-48), and by cosine similarity."""
import numpy as np
import pytest

from c0ven_b200 import MoELayer, synth
from oracle import oracle as O

pytestmark = pytest.mark.gpu

TYPES = [synth.Q8_0, synth.Q4_K, synth.Q6_K, synth.IQ3_S]
MAX_REL, MIN_COS = 1e-2, 0.9999   # the bar the layer is held to
INT_PATH_REL = 2e-3               # the integer-dot kernels: f32 summation order, and a code of h that rounds the other way


def errors(got, want):
    rel = float(np.abs(got - want).max() / np.abs(want).max())
    cos = float((got.astype(np.float64) * want).sum() / np.linalg.norm(got.astype(np.float64)) / np.linalg.norm(want.astype(np.float64)))
    return rel, cos


def check(layer, gpu, x, rel_bound=MAX_REL):
    T = x.shape[0]
    out = gpu.forward(x)
    ids, w, inv, tiles = gpu.route(T)
    ro, rids, rw, rinv, rtiles = O.moe_forward(layer, x)
    assert np.array_equal(ids, rids)
    assert np.array_equal(inv, rinv)
    assert np.array_equal(tiles, rtiles)
    assert np.allclose(w, rw, rtol=1e-5, atol=1e-7)
    rel, cos = errors(out, ro)
    assert rel <= rel_bound and cos >= MIN_COS, (rel, cos)
    return out


@pytest.mark.parametrize("t", TYPES)
def test_small_layer_every_row_count(t):
    layer = synth.make_layer(n_embd=512, n_ff=256, n_experts=32, n_used=4, gate_type=t, seed=t)
    gpu = MoELayer(layer, max_tokens=256, no_tensor=True)
    for T in (1, 2, 3, 4, 5, 7, 8, 9, 31, 32, 33, 63, 64, 65, 200):
        check(layer, gpu, synth.make_input(T, 512, seed=T), INT_PATH_REL)
    gpu.close()


def test_mixed_types_and_skew():
    """Gate and up Q4_K, down Q6_K, shared expert Q8_0, Zipf bias on the router: the sweep configuration's types."""
    layer = synth.make_layer(n_embd=512, n_ff=256, n_experts=64, n_used=10, gate_type=synth.Q4_K, down_type=synth.Q6_K,
                             shexp_gate_type=synth.Q8_0, shexp_down_type=synth.Q8_0, zipf_s=1.1, seed=5)
    gpu = MoELayer(layer, max_tokens=512, no_tensor=True)
    for T in (1, 4, 32, 256, 500):
        check(layer, gpu, synth.make_input(T, 512, seed=10 + T), INT_PATH_REL)
    ids = gpu.route(500)[0]
    cnt = np.bincount(ids.reshape(-1), minlength=64)
    assert cnt.max() > 3 * cnt.mean()
    gpu.close()


def test_general_row_lengths():
    """Sizes no specialised instantiation takes (the reference file's 2560 and 640 are of this kind)."""
    layer = synth.make_layer(n_embd=768, n_ff=1280, n_experts=32, n_used=3, gate_type=synth.Q4_K, down_type=synth.Q8_0, seed=8)
    gpu = MoELayer(layer, max_tokens=64, no_tensor=True)
    for T in (1, 9, 40):
        check(layer, gpu, synth.make_input(T, 768, seed=T), INT_PATH_REL)
    gpu.close()


def test_same_bits_twice_and_alone_or_batched():
    """Run twice: the same bits. A row gives the same ids alone or among others (core/tests/pack_test.cpp:121-141 in kind)."""
    layer = synth.make_layer(n_embd=512, n_ff=256, n_experts=32, n_used=4, gate_type=synth.IQ3_S, seed=21)
    gpu = MoELayer(layer, max_tokens=128, no_tensor=True)
    x = synth.make_input(100, 512, seed=2)
    a = gpu.forward(x).copy()
    ids_a, _, inv_a, _ = gpu.route(100)
    b = gpu.forward(x)
    ids_b, _, inv_b, _ = gpu.route(100)
    assert np.array_equal(a, b) and np.array_equal(ids_a, ids_b) and np.array_equal(inv_a, inv_b)
    gpu.forward(x[17:18])
    assert np.array_equal(gpu.route(1)[0][0], ids_a[17])
    gpu.close()


def test_near_ties_route_like_the_oracle():
    """Rows built so that several experts' logits are equal or one ulp apart: the ids still match (ties to the lower
    expert, route.h:33-38)."""
    layer = synth.make_layer(n_embd=512, n_ff=256, n_experts=32, n_used=4, gate_type=synth.Q8_0, seed=33)
    layer["router"][5] = layer["router"][2]          # experts 2 and 5 tie on every row
    layer["router"][9] = layer["router"][2]
    layer["router"][11] = np.nextafter(layer["router"][7], np.float32(np.inf))
    gpu = MoELayer(layer, max_tokens=128, no_tensor=True)
    check(layer, gpu, synth.make_input(100, 512, seed=4), INT_PATH_REL)
    x = np.zeros((3, 512), dtype=np.float32)         # all logits 0: experts 0..3, weights 1/4
    x[1, 0] = -0.0
    out = gpu.forward(x)
    ids, w, inv, tiles = gpu.route(3)
    ro, rids, rw, rinv, rtiles = O.moe_forward(layer, x)
    assert np.array_equal(ids, rids) and np.array_equal(inv, rinv) and np.array_equal(tiles, rtiles)
    assert np.array_equal(ids, np.tile(np.arange(4, dtype=np.int32), (3, 1)))
    assert np.allclose(w, 0.25) and np.all(out == 0) and np.all(ro == 0)
    gpu.close()


def test_swiglu_limit():
    layer = synth.make_layer(n_embd=512, n_ff=256, n_experts=32, n_used=4, gate_type=synth.Q4_K, seed=12, swiglu_limit=2.0)
    gpu = MoELayer(layer, max_tokens=32, no_tensor=True)
    check(layer, gpu, synth.make_input(20, 512, seed=1), INT_PATH_REL)
    gpu.close()


def test_bad_calls_are_refused():
    from c0ven_b200 import MoEError, _lib

    layer = synth.make_layer(n_embd=256, n_ff=256, n_experts=32, n_used=4, gate_type=synth.Q8_0, seed=1)
    gpu = MoELayer(layer, max_tokens=16)
    with pytest.raises(MoEError) as e:
        gpu.forward(synth.make_input(17, 256))
    assert e.value.status == _lib.MOE_BAD_ARGUMENT
    gpu.forward(synth.make_input(16, 256))
    gpu.close()


@pytest.mark.parametrize("t", TYPES)
def test_tensor_core_path_small_layer(t):
    """Every expert through the tcgen05 grouped GEMM (tensor_min_rows 1), then the default split between the two
    kinds of kernel, over row counts around the tile sizes (16, 64, 256)."""
    layer = synth.make_layer(n_embd=512, n_ff=256, n_experts=32, n_used=4, gate_type=t, zipf_s=1.1, seed=40 + t)
    for tm in (1, 0):
        gpu = MoELayer(layer, max_tokens=1100, tensor_min_rows=tm)
        for T in (1, 15, 16, 17, 63, 64, 65, 255, 256, 257, 1000):
            check(layer, gpu, synth.make_input(T, 512, seed=T))
        assert gpu.stats()["last_tensor_rows"] > 0
        gpu.close()


def test_tensor_core_path_mixed_types():
    layer = synth.make_layer(n_embd=512, n_ff=256, n_experts=64, n_used=10, gate_type=synth.Q4_K, down_type=synth.Q6_K,
                             shexp_gate_type=synth.Q8_0, shexp_down_type=synth.Q8_0, zipf_s=1.1, seed=6)
    gpu = MoELayer(layer, max_tokens=2048)
    for T in (32, 256, 2048):
        check(layer, gpu, synth.make_input(T, 512, seed=20 + T))
    gpu.close()


@pytest.fixture(scope="module")
def full_q8_0():
    """The benchmark shape: hidden 2048, FFN 512, 512 experts, top 10, Q8_0 (configuration 1)."""
    layer = synth.make_layer(gate_type=synth.Q8_0, seed=100)
    gpu = MoELayer(layer, max_tokens=64, no_tensor=True)
    yield layer, gpu
    gpu.close()


def test_full_shape_decode_q8_0(full_q8_0):
    layer, gpu = full_q8_0
    check(layer, gpu, synth.make_input(1, 2048, seed=7), INT_PATH_REL)
    check(layer, gpu, synth.make_input(32, 2048, seed=8), INT_PATH_REL)


@pytest.mark.parametrize("t", [synth.Q4_K, synth.IQ3_S])
def test_full_shape_ragged_batch(t):
    """512 experts with the Zipf bias, a ragged batch of runs {1, 8, 40, 100} (configuration 2's kind, fewer rows)."""
    layer = synth.make_layer(gate_type=t, zipf_s=1.1, seed=200 + t)
    gpu = MoELayer(layer, max_tokens=160, no_tensor=True)
    check(layer, gpu, synth.make_input(149, 2048, seed=9), INT_PATH_REL)
    gpu.close()
    gpu = MoELayer(layer, max_tokens=700, tensor_min_rows=16)   # the hot experts on the tensor cores, the tail on the integer dots
    check(layer, gpu, synth.make_input(620, 2048, seed=10))
    st = gpu.stats()
    assert 0 < st["last_tensor_rows"] < 620 * 11
    gpu.close()


def test_full_size_ragged3521_q4_k():
    """Configuration 2 at its full size: 3,521 rows as runs {1, 8, 512, 3000}, Q4_K, Zipf 1.1, every expert on the
    tile kernels. The routing of all 3,521 rows is compared bit for bit with the oracle's (ids, the pack permutation,
    the tiles); the outputs of a sample of rows from every run with the oracle's for those rows computed alone, which
    the oracle's per-token independence allows (core/tests/cpu_experts_test.cpp:240-275 in kind); and the first 100
    rows run as their own batch route the same."""
    layer = synth.make_layer(gate_type=synth.Q4_K, zipf_s=1.1, seed=0)
    T = 3521
    x = synth.make_input(T, 2048, seed=1)
    gpu = MoELayer(layer, max_tokens=T)
    out = gpu.forward(x)
    ids, w, inv, tiles = gpu.route(T)
    st = gpu.stats()
    assert st["last_tensor_rows"] >= T * 10   # 35,210 rows >= 1,280: every expert takes the tile kernels
    rl = O.router_logits(x, layer["router"], layer["shexp_gate_inp"], layer["router_bias"])
    rids, rw, _ = O.router_topk(rl, 10)
    assert np.array_equal(ids, rids)
    assert np.allclose(w, rw, rtol=1e-5, atol=1e-7)
    cnt, base, rinv, rtiles = O.pack(rids, 512)
    assert np.array_equal(inv, rinv) and np.array_equal(tiles, rtiles)
    assert sorted(inv.tolist()) == list(range(T * 10))
    sample = np.array([0, 1, 5, 8, 9, 100, 300, 520, 521, 1000, 2000, 3000, 3520])
    ref = O.moe_forward(layer, x[sample])[0]
    rel, cos = errors(out[sample], ref)
    assert rel <= MAX_REL and cos >= MIN_COS, (rel, cos)
    gpu.forward(x[:100])
    assert np.array_equal(gpu.route(100)[0], ids[:100])
    gpu.close()
