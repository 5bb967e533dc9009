"""The CPU oracle against what pins it: gguf-py's golden vectors, its own dequantisation in double, and the
reference's stated rules for routing and packing (kernels/models/qwen4exp/route.h:33-38, core/tests/topk_test.cpp:62-72,
core/tests/step_rows_test.cpp:40-58, core/tests/quant_test.cpp:67-81,108-120, core/tests/cpu_experts_test.cpp:240-275)."""
import numpy as np
import pytest

from c0ven_b200 import synth
from oracle import oracle as O

TYPES = [synth.Q8_0, synth.Q4_K, synth.Q6_K, synth.IQ3_S, synth.IQ4_NL, synth.IQ4_XS, synth.IQ3_XXS, synth.IQ2_S]
# Q2_0 is a type of the reference's fork of ggml: gguf-py has no decoder for it, so it is held to its stated rule.
ALL_TYPES = TYPES + [synth.Q2_0]


@pytest.mark.parametrize("t", ALL_TYPES)
def test_tables_match_shared_quant_h(t):
    assert O.block_values(t) == synth.BLOCK_VALUES[t]
    assert O.block_bytes(t) == synth.BLOCK_BYTES[t]
    assert O.vec_dot_type(t) == (O.Q8_0 if t in (synth.Q8_0, synth.IQ4_NL, synth.Q2_0) else O.Q8_K)


def test_q2_0_decodes_by_its_rule():
    """y = (q - 1) * d, four 2-bit codes a byte, value j in bits 2 (j mod 4) of byte j / 4 (docs/spec/QUANT_FORMATS.md:251-263)."""
    rng = np.random.default_rng(42)
    blocks = synth.random_blocks(synth.Q2_0, 50, rng)
    blocks[0, 2:] = 0
    blocks[1, 2:] = 255
    d = blocks[:, :2].copy().view(np.float16).astype(np.float32)
    codes = (blocks[:, 2:, None] >> np.array([0, 2, 4, 6], dtype=np.uint8)) & 3
    want = ((codes.reshape(50, 64).astype(np.float32) - 1) * d).reshape(-1)
    assert np.array_equal(O.dequantize(synth.Q2_0, blocks, want.size), want)


@pytest.mark.parametrize("t", TYPES)
def test_dequantize_equals_gguf_py(t, golden):
    blocks, want = golden[f"blocks_{t}"], golden[f"values_{t}"]
    got = O.dequantize(t, blocks, want.size)
    assert np.array_equal(got, want)  # integer decode and one rounding each: exact


def test_q8_0_quantiser_equals_gguf_py(golden):
    got = O.quantize(O.Q8_0, golden["q8_0_x"]).reshape(-1, 34)
    assert np.array_equal(got, golden["q8_0_blocks"])


def _q8k_fields(a):
    ab = a.reshape(-1, 292)
    d = ab[:, :4].copy().view(np.float32).reshape(-1)
    qs = ab[:, 4:260].view(np.int8)
    bs = ab[:, 260:].copy().view(np.int16).reshape(-1, 16)
    return d, qs, bs


def test_q8_K_quantiser_rule():
    rng = np.random.default_rng(5)
    x = (rng.standard_normal(256 * 6) * 3).astype(np.float32)
    x[256:512] = 0.0
    x[512] = -50.0  # the largest magnitude negative: d positive
    d, qs, bs = _q8k_fields(O.quantize(O.Q8_K, x))
    xb = x.reshape(-1, 256)
    for i in range(6):
        if not xb[i].any():
            assert d[i] == 0 and not qs[i].any()
            continue
        mx = xb[i][np.argmax(np.abs(xb[i]))]
        iscale = np.float32(-127.0) / np.float32(mx)
        want = np.minimum(127, np.rint(iscale * xb[i])).astype(np.int8)
        assert np.array_equal(qs[i], want)
        assert d[i] == np.float32(1.0) / iscale
        assert np.array_equal(bs[i], qs[i].astype(np.int32).reshape(16, 16).sum(-1))
    assert d[2] > 0 and d[0] * x[np.argmax(np.abs(xb[0]))] < 0


@pytest.mark.parametrize("t", ALL_TYPES)
@pytest.mark.parametrize("n", [256, 512, 2048])
def test_dot_against_own_dequantisation(t, n):
    rng = np.random.default_rng(100 + t + n)
    for _ in range(4):
        w = synth.random_blocks(t, n // synth.BLOCK_VALUES[t], rng)
        x = rng.standard_normal(n).astype(np.float32)
        at = O.vec_dot_type(t)
        a = O.quantize(at, x)
        dw = O.dequantize(t, w, n).astype(np.float64)
        if at == O.Q8_0:
            da = O.dequantize(O.Q8_0, a, n).astype(np.float64)
        else:
            d, qs, _ = _q8k_fields(a)
            da = (d[:, None].astype(np.float64) * qs).reshape(-1)
        got, want = O.vec_dot(t, w, a, n), float(dw @ da)
        assert abs(got - want) <= 1e-4 * np.abs(dw * da).sum()  # quant_test.cpp:120's bound; in practice ~1e-8


@pytest.mark.parametrize("t", ALL_TYPES)
def test_runs_layout_is_a_permutation(t):
    rng = np.random.default_rng(7)
    n = 40
    blocks = synth.random_blocks(t, n, rng)
    runs = O.to_runs(t, blocks)
    assert np.array_equal(np.sort(runs.reshape(-1)), np.sort(blocks.reshape(-1)))
    assert np.array_equal(O.from_runs(t, runs).reshape(blocks.shape), blocks)
    # The first run holds every block's quants, block k's at k * size (shared/quant.h:172-176).
    qoff, qsz = {synth.Q8_0: (2, 32), synth.Q4_K: (16, 128), synth.Q6_K: (0, 128), synth.IQ3_S: (2, 64),
                 synth.IQ4_NL: (2, 16), synth.IQ4_XS: (8, 128), synth.IQ3_XXS: (2, 64), synth.IQ2_S: (2, 32), synth.Q2_0: (2, 16)}[t]
    assert np.array_equal(runs.reshape(-1)[:n * qsz].reshape(n, qsz), blocks[:, qoff:qoff + qsz])


def test_router_logits_order_and_value():
    rng = np.random.default_rng(9)
    E, NE, T = 512, 24, 5
    x = rng.standard_normal((T, E)).astype(np.float32)
    W = (rng.standard_normal((NE, E)) * 0.02).astype(np.float32)
    g = (rng.standard_normal(E) * 0.02).astype(np.float32)
    bias = rng.standard_normal(NE).astype(np.float32)
    rl = O.router_logits(x, W, g, bias)
    want = np.empty((T, NE + 1), dtype=np.float32)
    Wall = np.concatenate([W, g[None]], 0)
    for t in range(T):
        for e in range(NE + 1):
            tot = None
            for s in range(8):
                p = np.float32(0)
                for k in range(s * E // 8, (s + 1) * E // 8):
                    # fused multiply-add: the product exact in double, one rounding
                    p = np.float32(np.float64(x[t, k]) * np.float64(Wall[e, k]) + np.float64(p))
                tot = p if tot is None else np.float32(tot + p)
            want[t, e] = tot if e == NE else np.float32(tot + bias[e])
    assert np.array_equal(rl, want)


def test_topk_rank_order_and_ties():
    NE, K = 64, 10
    rng = np.random.default_rng(11)
    rl = rng.standard_normal((6, NE + 1)).astype(np.float32)
    rl[1, :NE] = 0.25               # all equal: the lowest 10 experts, in order
    rl[2, 5] = rl[2, 40] = 9.0      # a tie at the top: 5 before 40
    rl[3, 7] = -0.0
    rl[3, 3] = 0.0
    rl[3, :NE][np.arange(NE) % 2 == 0] = -1.0  # many below; -0 (7) and +0 (3) tie, 3 first
    rl[3, 3] = 0.0
    ids, w, gs = O.router_topk(rl, K)
    for t in range(6):
        order = sorted(range(NE), key=lambda e: (-float(rl[t, e] + 0.0), e))[:K]
        assert list(ids[t]) == order
        p = np.exp(rl[t, order].astype(np.float64) - rl[t, :NE].max())
        assert np.allclose(w[t], p / p.sum(), rtol=2e-6)
        assert abs(w[t].sum() - 1) < 1e-6
    assert list(ids[1]) == list(range(10))
    assert list(ids[2][:2]) == [5, 40]
    assert np.allclose(gs, 1 / (1 + np.exp(-rl[:, NE].astype(np.float64))), rtol=1e-6)


def test_pack_is_a_stable_sort_with_tiles_of_64():
    rng = np.random.default_rng(13)
    NE, K, T = 16, 4, 300
    ids = np.stack([rng.permutation(NE)[:K] for _ in range(T)]).astype(np.int32)
    ids[:, 0] = 3  # a hot expert: 300 rows, tiles 64 x 4 + 44
    for t in range(T):
        if 3 in ids[t, 1:]:
            ids[t, 1:][ids[t, 1:] == 3] = 15 if 15 not in ids[t] else 14
    cnt, base, inv, tiles = O.pack(ids, NE)
    flat = ids.reshape(-1)
    order = np.argsort(flat, kind="stable")
    want_inv = np.empty_like(order)
    want_inv[order] = np.arange(order.size)
    assert np.array_equal(inv, want_inv.astype(np.uint32))
    assert np.array_equal(cnt, np.bincount(flat, minlength=NE))
    assert np.array_equal(base, np.concatenate([[0], np.cumsum(cnt)[:-1]]))
    # Tiles: experts ascending, an expert's tiles consecutive, counts 1..64 (shared/moe_tile.h:9-18).
    rows = 0
    for e, slot, start, count in tiles:
        assert slot == e and start == rows and 1 <= count <= 64
        assert np.all(flat[order[start:start + count]] == e)
        rows += count
    assert rows == T * K
    assert [c for e, _, _, c in tiles if e == 3] == [64, 64, 64, 64, 44]


@pytest.mark.parametrize("gt,dt", [(synth.Q8_0, synth.Q8_0), (synth.Q4_K, synth.Q6_K), (synth.IQ3_S, synth.IQ3_S)])
def test_compute_many_matches_single_token_and_double(gt, dt):
    """compute_many's token t has the bits of computing t alone (cpu_experts_test.cpp:240-275), and stays within the
    activation quantisation's error of the same sum on dequantised weights in double."""
    rng = np.random.default_rng(17)
    E, F, NX = 512, 256, 5
    ex = [(synth.random_matrix(gt, F, E, rng), synth.random_matrix(gt, F, E, rng), synth.random_matrix(dt, E, F, rng))
          for _ in range(NX)]
    x = rng.standard_normal((4, E)).astype(np.float32)
    jobs = []
    for t in range(4):
        for e in rng.permutation(NX)[:3]:
            jobs.append((*ex[e], t, float(rng.uniform(0.1, 0.5))))
    y = O.compute_many(gt, dt, E, F, jobs, x)
    for t in range(4):
        alone = O.compute_many(gt, dt, E, F, [(g, u, d, 0, w) for g, u, d, tok, w in jobs if tok == t], x[t:t + 1])
        assert np.array_equal(alone[0], y[t])
    deq = lambda m, ty, n: np.stack([O.dequantize(ty, r, n) for r in m]).astype(np.float64)
    ref = np.zeros((4, E))
    for g, u, d, tok, w in jobs:
        xv = x[tok].astype(np.float64)
        gg, uu = deq(g, gt, E) @ xv, deq(u, gt, E) @ xv
        ref[tok] += np.float32(w) * (deq(d, dt, F) @ (gg / (1 + np.exp(-gg)) * uu))
    assert np.abs(y - ref).max() / np.abs(ref).max() < 2e-2
    assert (y * ref).sum() / np.linalg.norm(y) / np.linalg.norm(ref) > 0.9995


def test_swiglu_limit():
    rng = np.random.default_rng(19)
    E, F = 256, 256
    g, u, d = (synth.random_matrix(synth.Q8_0, F, E, rng), synth.random_matrix(synth.Q8_0, F, E, rng),
               synth.random_matrix(synth.Q8_0, E, F, rng))
    for m in (g, u):  # larger scales so the limit bites
        m.reshape(-1, 34)[:, 0:2] = np.full((m.size // 34, 1), 0.02, np.float16).view(np.uint8).reshape(-1, 2)
    x = rng.standard_normal((1, E)).astype(np.float32)
    y0 = O.compute_many(synth.Q8_0, synth.Q8_0, E, F, [(g, u, d, 0, 1.0)], x)
    y1 = O.compute_many(synth.Q8_0, synth.Q8_0, E, F, [(g, u, d, 0, 1.0)], x, swiglu_limit=1.0)
    assert not np.allclose(y0, y1)
    deq = lambda m, n: np.stack([O.dequantize(synth.Q8_0, r, n) for r in m]).astype(np.float64)
    xa = O.dequantize(O.Q8_0, O.quantize(O.Q8_0, x[0]), E).astype(np.float64)
    gg, uu = np.minimum(deq(g, E) @ xa, 1.0), np.clip(deq(u, E) @ xa, -1.0, 1.0)
    h = (gg / (1 + np.exp(-gg)) * uu).astype(np.float32)
    ha = O.dequantize(O.Q8_0, O.quantize(O.Q8_0, h), F).astype(np.float64)
    assert np.abs(y1[0] - deq(d, F) @ ha).max() <= 1e-5 * np.abs(y1).max() + 1e-7  # experts_test.cpp:132


def test_layer_forward_consistent_with_its_parts():
    L = synth.make_layer(n_embd=512, n_ff=256, n_experts=32, n_used=4, gate_type=synth.Q4_K, zipf_s=1.1, seed=3)
    x = synth.make_input(70, 512)
    out, ids, w, inv, tiles = O.moe_forward(L, x)
    rl = O.router_logits(x, L["router"], L["shexp_gate_inp"], L["router_bias"])
    ids2, w2, gs = O.router_topk(rl, 4)
    assert np.array_equal(ids, ids2) and np.array_equal(w, w2)
    assert np.array_equal(inv, O.pack(ids, 32)[2])
    t = 11
    jobs = [(L["gate_exps"][e], L["up_exps"][e], L["down_exps"][e], 0, float(w[t, k])) for k, e in enumerate(ids[t])]
    moe = O.compute_many(synth.Q4_K, synth.Q4_K, 512, 256, jobs, x[t:t + 1])[0]
    sh = O.compute_many(synth.Q4_K, synth.Q4_K, 512, 256, [(L["gate_shexp"], L["up_shexp"], L["down_shexp"], 0, 1.0)],
                        x[t:t + 1])[0]
    assert np.array_equal(out[t], moe + gs[t] * sh)
    # Run twice: the same bits, whatever the threads did.
    assert np.array_equal(out, O.moe_forward(L, x)[0])
    # Skew: the bias makes a few experts take most rows.
    cnt = np.bincount(ids.reshape(-1), minlength=32)
    assert cnt.max() > 3 * cnt.mean()
