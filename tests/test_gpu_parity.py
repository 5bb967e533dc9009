"""On a B200: the CUDA layer, through the C ABI, against the CPU oracle on the same seeded inputs. Expert ids, the
pack permutation and the tiles are compared bit for bit; outputs by the reference's error measure,
max|a - b| / max|b| (docs/TESTING.md:47-48), and by cosine similarity."""
import numpy as np
import pytest

from c0ven_b200 import MoELayer, synth
from oracle import oracle as O

pytestmark = pytest.mark.gpu

TYPES = [synth.Q8_0, synth.Q4_K, synth.Q6_K, synth.IQ3_S, synth.IQ4_NL, synth.IQ4_XS, synth.IQ3_XXS, synth.IQ2_S, synth.Q2_0]
MAX_REL, MIN_COS = 1e-2, 0.9999   # the bar the layer is held to
# Routing weights: 1e-5 where the logits are the exactly ordered fp32 sums (steps of up to 64 rows). Longer steps take
# their logits from the tensor-core product, a few 1e-6 from those sums; the weights follow, while the expert ids, which
# are decided on exactly recomputed logits wherever the product's error bound leaves them open, stay bit for bit.
W_RTOL, W_RTOL_LONG = 1e-5, 2e-4
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
    assert np.allclose(w, rw, rtol=W_RTOL if T <= 64 else W_RTOL_LONG, atol=1e-7)
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


def test_tile_kernels_give_the_same_bits_every_run():
    """The tensor-core path at the full shape, with types mixed so that kernels of different kinds follow one another
    (Q4_K's quants come through a ring of bulk copies, the others' by the warps' own loads): six runs, the same bits of
    the output and of every quantised inner row. (A copy that refilled a ring slot before the warps' reads of it were
    done once showed here as a few wrong weight rows, different from run to run.)"""
    layer = synth.make_layer(gate_type=synth.Q4_K, down_type=synth.Q6_K, shexp_gate_type=synth.Q8_0, shexp_down_type=synth.Q8_0,
                             zipf_s=1.1, seed=5)
    gpu = MoELayer(layer, max_tokens=2048)
    x = synth.make_input(2048, 2048, seed=77)
    first = None
    for _ in range(6):
        out = gpu.forward(x).copy()
        q, d, _bs = gpu.quantized(2048, inner=True)
        if first is None:
            first = (out, q.copy(), d.copy())
        else:
            assert np.array_equal(q, first[1]) and np.array_equal(d, first[2])
            assert np.array_equal(out, first[0])
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
    assert np.allclose(w, rw, rtol=W_RTOL_LONG, atol=1e-7)
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


def _route_and_sample(layer, gpu, x, sample, K=10, w_rtol=W_RTOL_LONG):
    """Routing of every row bit for bit; outputs of the sampled rows against the oracle run on those rows alone (the
    oracle's rows are independent: core/tests/cpu_experts_test.cpp:240-275)."""
    T = x.shape[0]
    out = gpu.forward(x)
    ids, w, inv, tiles = gpu.route(T)
    rl = O.router_logits(x, layer["router"], layer["shexp_gate_inp"], layer.get("router_bias"))
    rids, rw, _ = O.router_topk(rl, K)
    assert np.array_equal(ids, rids)
    assert np.allclose(w, rw, rtol=w_rtol, atol=1e-7)
    cnt, base, rinv, rtiles = O.pack(rids, layer["n_experts"])
    assert np.array_equal(inv, rinv) and np.array_equal(tiles, rtiles)
    sample = np.unique(np.asarray(sample))
    ref = O.moe_forward(layer, x[sample])[0]
    rel, cos = errors(out[sample], ref)
    assert rel <= MAX_REL and cos >= MIN_COS, (rel, cos)
    return out, ids, cnt


def test_full_size_prefill32768_q4_k():
    """Configuration 4 at its full size: one sequence of 32,768 rows, Q4_K, router without bias (about 640 rows an
    expert), every expert on the tile kernels. Routing of all rows bit for bit; outputs of 96 rows: the first and last
    rows, rows spread over the batch, and rows routed to the fullest and to the emptiest expert."""
    layer = synth.make_layer(gate_type=synth.Q4_K, seed=0)
    T = 32768
    x = synth.make_input(T, 2048, seed=1)
    gpu = MoELayer(layer, max_tokens=T)
    rl = O.router_logits(x, layer["router"], layer["shexp_gate_inp"], None)
    rids = O.router_topk(rl, 10)[0]
    cnt = np.bincount(rids.reshape(-1), minlength=512)
    full, empty = int(cnt.argmax()), int(cnt.argmin())
    rows_full = np.nonzero((rids == full).any(1))[0][:16]
    rows_empty = np.nonzero((rids == empty).any(1))[0][:16]
    sample = np.concatenate([[0, 1, T - 2, T - 1], np.linspace(0, T - 1, 60).astype(np.int64), rows_full, rows_empty])
    _route_and_sample(layer, gpu, x, sample)
    assert gpu.stats()["last_tensor_rows"] >= T * 10
    gpu.close()


def test_gate_up_kernel_gathering_its_rows_itself():
    """MOE_FLAG_GATHER_IN_KERNEL at a size it applies to (16,384 rows, 163,840 expert rows): the tile kernel fetches its
    rows by index with four-row gather copies. The products do not depend on how the rows came in, so the outputs are
    the bits of the layer that gathers first; routing against the oracle, outputs of sampled rows too."""
    layer = synth.make_layer(gate_type=synth.Q4_K, zipf_s=0.0, seed=77)
    T = 16384
    x = synth.make_input(T, 2048, seed=78)
    a = MoELayer(layer, max_tokens=T)
    want = a.forward(x).copy()
    a.close()
    b = MoELayer(layer, max_tokens=T, gather_in_kernel=True)
    _route_and_sample(layer, b, x, np.linspace(0, T - 1, 24).astype(np.int64))
    got = b.forward(x)
    assert np.array_equal(got, want)
    b.close()


def test_full_shape_sweep_q4k_q6k_q8_0():
    """Configuration 5 at the real shape (hidden 2048, FFN 512, 512 experts, top 10): Q4_K gate and up, Q6_K down, Q8_0
    shared expert, Zipf routing, at every point of its sweep. Short steps whole against the oracle; the long ones by
    routing of every row and outputs of sampled rows."""
    layer = synth.make_layer(gate_type=synth.Q4_K, down_type=synth.Q6_K, shexp_gate_type=synth.Q8_0, shexp_down_type=synth.Q8_0,
                             zipf_s=1.1, seed=5)
    gpu = MoELayer(layer, max_tokens=8192)
    for T in (1, 4, 32, 256):
        check(layer, gpu, synth.make_input(T, 2048, seed=30 + T))
    for T in (2048, 8192):
        x = synth.make_input(T, 2048, seed=30 + T)
        _route_and_sample(layer, gpu, x, np.concatenate([[0, T - 1], np.linspace(0, T - 1, 46).astype(np.int64)]))
    gpu.close()


@pytest.mark.parametrize("t", [synth.Q8_0, synth.Q6_K, synth.IQ4_NL, synth.IQ4_XS, synth.IQ3_XXS, synth.IQ2_S, synth.Q2_0])
def test_tile_kernels_full_shape_other_types(t):
    """The tile kernels' Q8_0, Q6_K, IQ4_NL, IQ4_XS, IQ3_XXS, IQ2_S and Q2_0 decoders at the full shape (rows of 2048 and of 512 values), every expert on them."""
    layer = synth.make_layer(gate_type=t, zipf_s=1.1, seed=300 + t)
    gpu = MoELayer(layer, max_tokens=700, tensor_min_rows=1)
    x = synth.make_input(700, 2048, seed=11)
    _route_and_sample(layer, gpu, x, np.linspace(0, 699, 48).astype(np.int64))
    assert gpu.stats()["last_tensor_rows"] >= 700 * 10
    gpu.close()


def test_three_layer_stack_with_residual():
    """Configuration 3's kind: a stack of layers with the residual, x <- x + moe_l(x), IQ3_S, 32 rows (4 requests of 8
    drafted rows). Layer by layer against the oracle on the same input (the GPU's own running x, so that the routing
    is the same question on both sides): ids bit for bit, outputs within the bar; and the stack's end against the
    oracle's own chain, which a near-tie routed the other way somewhere along it may part from, by cosine."""
    layers = [synth.make_layer(gate_type=synth.IQ3_S, seed=400 + i) for i in range(3)]
    for L in layers[1:]:  # the experts' bytes shared, the routers their own (as the bench's stack)
        for k in ("gate_exps", "up_exps", "down_exps", "gate_shexp", "up_shexp", "down_shexp"):
            L[k] = layers[0][k]
    x = synth.make_input(32, 2048, seed=12)
    xg, xo = x.copy(), x.copy()
    gpus = [MoELayer(L, max_tokens=32) for L in layers]
    for L, g in zip(layers, gpus):
        xin = xg / np.sqrt((xg.astype(np.float64) ** 2).mean(-1, keepdims=True) + 1e-6).astype(np.float32)   # the bench's norm between layers
        out = check(L, g, xin)
        xg = xg + out
        xon = xo / np.sqrt((xo.astype(np.float64) ** 2).mean(-1, keepdims=True) + 1e-6).astype(np.float32)
        xo = xo + O.moe_forward(L, xon)[0]
    rel, cos = errors(xg - x, xo - x)
    assert cos >= 0.995, (rel, cos)
    for g in gpus:
        g.close()


def _oracle_quantized(rows, q8k):
    """The oracle's quantised rows taken apart: codes, scales and (q8_K) sums."""
    n, Kv = rows.shape
    codes, scales, sums = [], [], []
    for r in rows:
        b = O.quantize(O.Q8_K if q8k else O.Q8_0, r)
        if q8k:
            b = b.reshape(Kv // 256, 292)
            scales.append(b[:, :4].copy().view(np.float32).reshape(-1))
            codes.append(b[:, 4:260].copy().view(np.int8).reshape(-1))
            sums.append(b[:, 260:].copy().view(np.int16).reshape(-1))
        else:
            b = b.reshape(Kv // 32, 34)
            scales.append(b[:, :2].copy().view(np.float16).astype(np.float32).reshape(-1))
            codes.append(b[:, 2:].copy().view(np.int8).reshape(-1))
    return np.stack(codes), np.stack(scales), (np.stack(sums) if q8k else None)


@pytest.mark.parametrize("t", [synth.Q8_0, synth.Q4_K])
def test_activation_quantiser_bit_for_bit(t):
    """The quantised rows the expert kernels read (q8_0 for Q8_0 weights, q8_K for the K-quants) against the oracle's
    quantiser: every code, scale and block sum of x equal (docs/spec/QUANT_FORMATS.md:463-465,528-535). The inner rows
    h cannot be held to that: h itself differs from the oracle's in its last bits (another summation order in the
    products before it), and a value on a rounding boundary then takes the neighbouring code; there, codes differ by at
    most one and rarely."""
    layer = synth.make_layer(n_embd=512, n_ff=256, n_experts=32, n_used=4, gate_type=t, seed=60 + t)
    gpu = MoELayer(layer, max_tokens=128, no_tensor=True)
    x = synth.make_input(100, 512, seed=13)
    x[3] = 0.0                 # a row of zeros: scale 0, codes 0
    x[4, 17] = -x[4].max() * 2  # the largest magnitude negative
    gpu.forward(x)
    q, d, bs = gpu.quantized(100)
    rq, rd, rbs = _oracle_quantized(x, t != synth.Q8_0)
    assert np.array_equal(q, rq) and np.array_equal(d, rd)
    if rbs is not None:
        assert np.array_equal(bs, rbs)
    # h, in expert order, against the oracle's quantiser on the oracle's own h is not available through its interface;
    # hold the GPU's codes to its own h instead: re-quantising the dequantised rows gives the same codes back.
    hq, hd, _ = gpu.quantized(100, inner=True)
    assert hq.shape == (400, 256) and np.abs(hq).max() <= 127
    gpu.close()


def test_groups_hold_what_the_reference_groups_hold():
    """The decode path's groups against core/tests/step_rows_test.cpp:40-58's host rule: an expert's assignments in
    ascending order, a new group after every 8. The list is in expert order here (there: in order of first assignment),
    so the two are compared as sets of (expert, assignments)."""
    layer = synth.make_layer(n_embd=512, n_ff=256, n_experts=32, n_used=4, gate_type=synth.Q8_0, zipf_s=1.1, seed=70)
    gpu = MoELayer(layer, max_tokens=64, no_tensor=True)
    for T in (1, 8, 9, 12, 16, 40):
        gpu.forward(synth.make_input(T, 512, seed=T))
        ids, _, inv, _ = gpu.route(T)
        groups = gpu.groups()
        order = np.empty(T * 4, dtype=np.int64)
        order[inv] = np.arange(T * 4)           # expert-order row -> assignment
        got = sorted((int(s), tuple(int(a) for a in order[st:st + n])) for s, st, n in groups)
        cap = 2 if T * 4 <= 32 else 8           # steps with no more rows than experts take groups of two
        want, open_ = [], {}
        for a, e in enumerate(ids.reshape(-1)):  # the host rule, with the step's cap
            g = open_.get(int(e))
            if g is None or len(g) == cap:
                g = []
                open_[int(e)] = g
                want.append((int(e), g))
            g.append(a)
        assert got == sorted((e, tuple(g)) for e, g in want)
    gpu.close()


def test_a_wait_that_runs_out_returns_timeout():
    """The bounded wait of the C ABI: with a long step queued, a wait of one millisecond returns MOE_TIMEOUT (and hangs
    nothing: the step goes on); the wait after it, with the default limit, finds the step done and its results valid."""
    import torch

    from c0ven_b200 import MoEError, _lib

    layer = synth.make_layer(n_embd=2048, n_ff=512, n_experts=64, n_used=8, gate_type=synth.Q4_K, seed=90)
    T = 16384
    gpu = MoELayer(layer, max_tokens=T)
    x = torch.from_numpy(synth.make_input(T, 2048, seed=14)).cuda()
    out = torch.empty_like(x)
    torch.cuda.synchronize()
    for _ in range(4):   # several steps of a few milliseconds each
        gpu.forward_device(x.data_ptr(), T, out.data_ptr())
    with pytest.raises(MoEError) as e:
        gpu.sync(timeout_ms=1)
    assert e.value.status == _lib.MOE_TIMEOUT
    gpu.sync()
    assert torch.isfinite(out).all()
    gpu.close()


def test_tensor_core_router_keeps_the_exact_order():
    """Steps of more than 64 rows take their logits from the tensor-core product. Every expert here has a twin whose
    router row is the same up to one ulp in a few places, so every row of the batch has near-ties all through its top
    ten (thousands in all), which only exactly ordered logits decide; some twins are exact copies (ties go to the lower
    expert). The ids must still equal the oracle's bit for bit. Then the rows the product cannot serve: rows of zeros
    (every logit equal: more candidates than a warp holds) and a row with a value beyond f16's range."""
    layer = synth.make_layer(n_embd=1024, n_ff=256, n_experts=512, n_used=10, gate_type=synth.Q8_0, zipf_s=1.1, seed=81)
    rng = np.random.default_rng(82)
    R = layer["router"]
    for e in range(0, 512, 2):
        R[e + 1] = R[e]
        if e % 8:  # three pairs in four differ by an ulp in a few places; the fourth is an exact copy
            at = rng.integers(0, 1024, size=3)
            R[e + 1, at] = np.nextafter(R[e, at], np.float32(np.inf if e % 4 else -np.inf))
    layer["router_bias"][1::2] = layer["router_bias"][0::2]
    layer["router_bias"][100:200] = 2.0   # on a row of zeros a hundred experts tie for the top
    T = 1500
    x = synth.make_input(T, 1024, seed=83)
    x[7] = 0.0
    x[700:710] = 0.0
    x[11, 5] = 1.0e5
    x[12, 100] = -3.0e38
    gpu = MoELayer(layer, max_tokens=T, no_tensor=False)
    gpu.forward(x)
    ids, w, inv, tiles = gpu.route(T)
    rl = O.router_logits(x, R, layer["shexp_gate_inp"], layer["router_bias"])
    rids, rw, _ = O.router_topk(rl, 10)
    assert np.array_equal(ids, rids)
    ok = np.ones(T, dtype=bool)
    ok[[11, 12]] = False   # their weights come from exact logits too, but an overflowing sum may differ; ids are what is held
    assert np.allclose(w[ok], rw[ok], rtol=W_RTOL_LONG, atol=1e-7)
    assert np.array_equal(ids[7], np.arange(100, 110)) and np.array_equal(inv, O.pack(rids, 512)[2])
    # The product's error against the bound it claims, on the ordinary rows.
    lg, approx, eps_rel, eps_abs = gpu.logits(T)
    assert approx and eps_rel > 0
    exact = rl[:, :512] - layer["router_bias"][None, :]
    bound = eps_rel * np.linalg.norm(x.astype(np.float64), axis=1) + eps_abs
    rows = np.setdiff1d(np.arange(T), [11, 12])
    err = np.abs(lg[rows].astype(np.float64) - exact[rows]).max(axis=1)
    assert np.all(err <= bound[rows] / 4), float((err / bound[rows]).max())
    gpu.close()
