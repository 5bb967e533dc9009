"""On a B200: the engine ABI end to end over a small MoE-only model written as a GGUF file. Four slots are admitted and
driven through engine_submit / engine_poll the way configuration 3 is shaped (a plan carries a piece of 8 rows for each
of 4 slots: one packed ragged batch of 32 rows; later plans carry decode rows beside a longer piece). The hidden rows a
plan's batch ends with must equal, bit for bit, the same stack run through the layer-level C ABI (layers from the same
file, the library's norm kernel, the residual added by the combine: x <- x + moe_l(rmsnorm_l(x))), which the parity tests
hold to the oracle layer by layer; against the oracle's own chain they are compared loosely, since a near-tie routed
the other way in a later layer parts the two chains. Tokens must be the arg-max of those rows against the embedding;
events, timing records and counters must tell the same story."""
import numpy as np
import pytest

from c0ven_b200 import synth
from oracle import oracle as O

pytestmark = pytest.mark.gpu
pytest.importorskip("gguf")

E_, F_, NE, K, VOCAB, NL = 1024, 256, 64, 6, 300, 4


@pytest.fixture(scope="module")
def model(tmp_path_factory):
    rng = np.random.default_rng(700)
    layers = [synth.make_layer(n_embd=E_, n_ff=F_, n_experts=NE, n_used=K, gate_type=synth.IQ3_S, zipf_s=0.0, seed=700 + i) for i in range(NL)]
    embd = rng.standard_normal((VOCAB, E_)).astype(np.float32)
    norms = [(1.0 + 0.1 * rng.standard_normal(E_)).astype(np.float32) for _ in range(NL)]
    path = tmp_path_factory.mktemp("engine") / "moe_only.gguf"
    synth.write_gguf(path, layers, token_embd=embd, ffn_norms=norms)
    return path, layers, embd, norms


def oracle_stack(layers, norms, x):
    """x <- x + moe_l(rmsnorm_l(x)) with the CPU oracle; also every layer's expert ids."""
    ids = []
    for L, g in zip(layers, norms):
        xn = (x / np.sqrt((x.astype(np.float64) ** 2).mean(-1, keepdims=True) + 1e-6) * g).astype(np.float32)
        out, lid = O.moe_forward(L, xn)[:2]
        ids.append(lid)
        x = x + out
    return x, ids


def run_layer_stack(path, norms, x):
    import torch

    from c0ven_b200 import MoELayer
    from c0ven_b200.layer import GgufFile, rmsnorm_rows_device

    f = GgufFile(path)
    T = x.shape[0]
    xd = torch.from_numpy(np.ascontiguousarray(x)).cuda()
    xn = torch.empty_like(xd)
    gs = [torch.from_numpy(g).cuda() for g in norms]
    torch.cuda.synchronize()
    for i, g in enumerate(gs):
        L = MoELayer.from_gguf(f, i, max_tokens=128)
        rmsnorm_rows_device(xd.data_ptr(), g.data_ptr(), T, x.shape[1], 1e-6, xn.data_ptr(), L.stream)
        L.forward_residual_device(xn.data_ptr(), T, xd.data_ptr(), xd.data_ptr())
        L.sync()
        L.close()
    f.close()
    return xd.cpu().numpy()


def test_four_slots_of_eight_rows_one_batch_a_plan(model):
    from c0ven_b200 import engine as EN

    path, layers, embd, norms = model
    rng = np.random.default_rng(1)
    eng = EN.Engine(path, slots=4, max_ctx=256, prompt_chunk=128, checkpoints=1)
    assert eng.info.api_version == 23 and eng.info.slots == 4 and eng.info.vocab == VOCAB and eng.info.experts_per_layer == NE
    assert eng.info.max_step_rows == 128 and eng.info.cards == 1
    prompts = [rng.integers(0, VOCAB, size=n).tolist() for n in (16, 8, 20, 9)]
    for s, p in enumerate(prompts):
        eng.admit(s, p, max_tokens=3)
    with pytest.raises(EN.EngineError) as e:
        eng.admit(0, prompts[0])
    assert e.value.status == EN.BUSY
    # Plan 1: a piece of 8 rows for each of the 4 slots: one batch of 32 rows, four runs.
    eng.submit(pieces=[(s, 8) for s in range(4)])
    ev = eng.run_until_step(1)
    hidden, runs = eng.read_batch(E_)
    assert runs == [(8, 0, 0, 0), (8, 0, 1, 8), (8, 0, 2, 16), (8, 0, 3, 24)] and hidden.shape == (32, E_)
    toks = np.concatenate([p[:8] for p in prompts])
    assert np.array_equal(hidden, run_layer_stack(path, norms, embd[toks]))
    want, _ = oracle_stack(layers, norms, embd[toks])
    cos = float((hidden.astype(np.float64) * want).sum() / np.linalg.norm(hidden.astype(np.float64)) / np.linalg.norm(want.astype(np.float64)))
    assert cos >= 0.99, cos
    kinds = [(k, s, v) for k, s, t, v in ev]
    assert (EN.EVENT_PROMPT, 0, 8) in kinds and (EN.EVENT_PROMPT, 3, 8) in kinds
    # slot 1's prompt (8 tokens) ended in this plan: its first token is the arg-max of its last row against the embedding
    tok1 = [t for k, s, t, v in ev if k == EN.EVENT_TOKEN and s == 1]
    assert tok1 == [int(np.argmax(embd @ hidden[15]))]
    assert kinds[-1] == (EN.EVENT_STEP, 0, 1)
    # Plan 2: slot 1 decodes (its own token) beside pieces for the others: 1 + 8 + 12 + 1 rows in one batch.
    eng.submit(decode=[1], pieces=[(0, 8), (2, 0), (3, 0)])
    ev = eng.run_until_step(2)
    hidden, runs = eng.read_batch(E_)
    assert runs == [(8, 8, 0, 0), (12, 8, 2, 8), (1, 8, 3, 20), (1, 8, 1, 21)]
    toks = np.concatenate([prompts[0][8:16], prompts[2][8:20], prompts[3][8:9], tok1])
    assert np.array_equal(hidden, run_layer_stack(path, norms, embd[toks]))
    got_tokens = {s: t for k, s, t, v in ev if k == EN.EVENT_TOKEN}
    assert set(got_tokens) == {0, 1, 2, 3}   # every prompt ended in this plan, and slot 1 wrote its second token
    for s, row in ((0, 7), (2, 19), (3, 20), (1, 21)):
        assert got_tokens[s] == int(np.argmax(embd @ hidden[row]))
    # Plans 3 and 4: all four decode together; max_tokens 3 ends slot 1 first, then the others.
    eng.submit(decode=[0, 1, 2, 3])
    ev = eng.run_until_step(3)
    done = [(s, v) for k, s, t, v in ev if k == EN.EVENT_DONE]
    assert done == [(1, 2)]   # ENGINE_DONE_LENGTH
    eng.submit(decode=[0, 1, 2, 3])
    ev = eng.run_until_step(4)
    assert sorted(s for k, s, t, v in ev if k == EN.EVENT_DONE) == [0, 2, 3]
    _, runs = eng.read_batch(E_)
    assert [r[2] for r in runs] == [0, 2, 3]   # slot 1 was done: it brought no row
    # Timing records: one per piece and one for a plan's decode rows; counters add up.
    tm = eng.timing()
    assert [(k, p, r) for k, p, r, *_ in tm] == [(1, 1, 8)] * 4 + [(1, 2, 8), (1, 2, 12), (1, 2, 1), (2, 2, 1), (2, 3, 4), (2, 4, 3)]
    assert all(t[5] > t[4] for t in tm)
    st = eng.stats()
    assert st["plans"] == 4 and st["prompt_rows"] == 53 and st["step_rows"] == 8 and st["experts_cached"] == NE
    # A page change that leaves a gap is refused, as the reference refuses it; a consistent one is accepted.
    with pytest.raises(EN.EngineError) as e:
        eng.submit(pages=[(0, 5, 1, 0, 0)])
    assert e.value.status == EN.BAD_ARGUMENT
    eng.submit(pages=[(0, 0, 1, 0, 0), (0, 1, 2, 0, 0)])
    eng.run_until_step(5)
    # Checkpoint, release, admit again, restore: the slot continues after the checkpoint's tokens.
    eng.release(1)
    eng.admit(1, prompts[0], max_tokens=1)
    eng.submit(pieces=[(1, 8)])
    eng.run_until_step(6)
    eng.checkpoint(1, 0)
    eng.release(1)
    eng.admit(1, prompts[0], max_tokens=1)
    eng.restore(1, 0)
    eng.submit(pieces=[(1, 0)])
    eng.run_until_step(7)
    _, runs = eng.read_batch(E_)
    assert runs == [(8, 8, 1, 0)]
    # Sleep is refused while a slot is admitted; after release it frees the GPU, and wake loads the file again.
    with pytest.raises(EN.EngineError) as e:
        eng.sleep()
    assert e.value.status == EN.BUSY
    for s in range(4):
        eng.release(s)
    eng.sleep()
    with pytest.raises(EN.EngineError):
        eng.admit(0, prompts[0])
    eng.wake()
    eng.admit(0, prompts[1], max_tokens=1)
    eng.submit(pieces=[(0, 0)])
    ev = eng.run_until_step(8)
    assert [t for k, s, t, v in ev if k == EN.EVENT_TOKEN] == tok1   # the same prompt gives the same token after a wake
    eng.close()


def test_cards_lists_the_gpus():
    import ctypes

    from c0ven_b200 import engine as EN

    n = ctypes.c_uint32(0)
    cards = (EN.Card * 8)()
    assert EN.lib().engine_cards(cards, 8, ctypes.byref(n)) == EN.OK and n.value >= 1
    assert b"NVIDIA" in cards[0].name and cards[0].memory > 100 << 30 and cards[0].xe_cores >= 100
