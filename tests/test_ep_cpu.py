"""Expert parallel on two CPU ranks (gloo): the exchange logic of c0ven_b200.ep (split sizes, the two all-to-alls,
destination order, results back in place) with a CPU stand-in for the GPU stages. Each rank's outputs must be the
bits the oracle gives for that rank's rows on one process. Failures are made on the host: a stage that raises on one
rank, a rank that would receive more rows than it has room for, a rank that never joins a collective."""
import datetime
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from ep_common import run_ranks  # noqa: E402

from c0ven_b200 import ep, synth  # noqa: E402


def _init(rank, world, port, seconds=60):
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=seconds))


def _layer():
    return synth.make_layer(n_embd=256, n_ff=256, n_experts=32, n_used=4, gate_type=synth.Q4_K, zipf_s=1.1, seed=3)


def _worker(rank, world, port, q, T, by_token):
    from ep_common import OracleStages
    from oracle import oracle as O

    _init(rank, world, port)
    try:
        layer = _layer()
        x = synth.make_input(T[rank], 256, seed=10 + rank)
        moe = ep.ExpertParallelMoE(OracleStages(layer, rank, world), by_token=by_token)
        out = moe.forward(torch.from_numpy(x)).numpy()
        ref = O.moe_forward(layer, x)[0]
        rel = float(np.abs(out - ref).max() / np.abs(ref).max())
        q.put((rank, bool(np.array_equal(out, ref)), moe.sent_rows, moe.received_rows, rel))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("T", [(37, 5), (1, 64)])
def test_two_ranks_give_the_single_process_bits(T):
    """One row per assignment: each rank's outputs are the single process's bits."""
    res = run_ranks(_worker, 2, (T, False))
    assert all(r[1] for r in res)
    # What one rank sent to the other is what the other received from it.
    assert res[0][2] == res[1][3] and res[1][2] == res[0][3]


@pytest.mark.parametrize("world,T", [(2, (37, 5)), (4, (9, 1, 30, 2)), (8, (5, 1, 12, 3, 8, 2, 7, 4))])
def test_one_row_per_token_and_gpu(world, T):
    """One row per (token, GPU) out and one partial sum back: the outputs agree with the single process's to f32
    rounding (the sum over a token's experts is taken GPU by GPU), and fewer rows cross than there are assignments."""
    res = run_ranks(_worker, world, (T, True))
    assert all(r[4] <= 1e-5 for r in res), [r[4] for r in res]
    assert sum(r[2] for r in res) == sum(r[3] for r in res)          # rows sent = rows received, over all ranks
    assert sum(r[2] for r in res) < sum(T) * 4                        # fewer than one a (token, expert)


def _worker_stage_fails(rank, world, port, q, where, by_token):
    """Rank 1's stage raises in the middle of a step. Rank 0 must still leave the step (its collectives are all
    entered by rank 1 too, which raises only after them), and the step after that must work on both."""
    from ep_common import OracleStages

    _init(rank, world, port, seconds=30)
    try:
        st = OracleStages(_layer(), rank, world)
        real = getattr(st, where)
        calls = {"n": 0}

        def failing(*a):
            calls["n"] += 1
            if rank == 1 and calls["n"] == 1:
                raise RuntimeError("injected: the stage failed")
            return real(*a)

        setattr(st, where, failing)
        moe = ep.ExpertParallelMoE(st, by_token=by_token)
        x = torch.from_numpy(synth.make_input(9, 256, seed=rank))
        first = "ok"
        try:
            moe.forward(x)
        except RuntimeError as e:
            first = str(e)
        second = "ok"
        try:
            moe.forward(x)
        except RuntimeError as e:  # pragma: no cover
            second = str(e)
        q.put((rank, first, second))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("where,by_token", [("gather", False), ("experts", False), ("dispatch", True), ("experts_partial", True)])
def test_a_stage_that_fails_on_one_rank_does_not_strand_the_other(where, by_token):
    res = run_ranks(_worker_stage_fails, 2, (where, by_token), timeout=90)
    assert res[0][1] == "ok" and "injected" in res[1][1]
    assert res[0][2] == "ok" and res[1][2] == "ok"


def _worker_too_many_rows(rank, world, port, q):
    from ep_common import OracleStages

    _init(rank, world, port, seconds=30)
    try:
        st = OracleStages(_layer(), rank, world)
        st.max_expert_rows = 8   # far fewer than 2 x 20 rows x 4 experts can bring
        moe = ep.ExpertParallelMoE(st)
        try:
            moe.forward(torch.from_numpy(synth.make_input(20, 256, seed=rank)))
            q.put((rank, "ok"))
        except RuntimeError as e:
            q.put((rank, str(e)))
    finally:
        dist.destroy_process_group()


def test_every_rank_refuses_a_step_one_rank_has_no_room_for():
    res = run_ranks(_worker_too_many_rows, 2, timeout=90)
    assert all("max_expert_rows" in msg for _, msg in res)
    assert res[0][1] == res[1][1]   # the same message: the same decision, taken from the same gathered counts


def _worker_lost_peer(rank, world, port, q):
    """Rank 1 leaves before the step (between steps, nothing in flight). Rank 0's first collective ends with an error
    after the process group's short timeout instead of waiting for ever."""
    from ep_common import OracleStages

    _init(rank, world, port, seconds=5)
    if rank == 1:
        q.put((rank, "left"))
        return
    moe = ep.ExpertParallelMoE(OracleStages(_layer(), rank, world))
    t0 = datetime.datetime.now()
    try:
        moe.forward(torch.from_numpy(synth.make_input(4, 256, seed=0)))
        q.put((rank, "ok"))
    except Exception as e:  # noqa: BLE001
        q.put((rank, f"error after {(datetime.datetime.now() - t0).total_seconds():.0f} s: {type(e).__name__}"))


def test_a_lost_peer_ends_the_collective_with_an_error():
    res = run_ranks(_worker_lost_peer, 2, timeout=120)
    assert res[1][1] == "left" and res[0][1].startswith("error")


def test_balanced_order_spreads_a_zipf_load():
    """Contiguous ownership under the benchmark's Zipf bias leaves the busiest of 8 GPUs with nearly twice the mean
    load; dealing the experts by their counts brings it within a few percent, and interleaving alone most of the way."""
    rng = np.random.default_rng(0)
    bias = synth.zipf_bias(512, 1.1, rng)
    logits = rng.standard_normal((4000, 512)).astype(np.float32) * 0.9 + bias
    ids = np.argsort(-logits, axis=1)[:, :10]
    counts = np.bincount(ids.reshape(-1), minlength=512)

    def worst(order):
        per_gpu = counts[order].reshape(8, 64).sum(1)
        return per_gpu.max() / per_gpu.mean()

    assert worst(np.arange(512)) > 1.4
    bal = ep.balanced_order(counts, 8)
    assert sorted(bal.tolist()) == list(range(512))
    assert worst(bal) <= 1.05
    assert worst(ep.interleaved_order(512, 8)) < worst(np.arange(512))
    layer = synth.make_layer(n_embd=256, n_ff=256, n_experts=32, n_used=4, gate_type=synth.Q8_0, seed=9)
    re = ep.reordered(layer, ep.interleaved_order(32, 4))
    assert np.array_equal(re["router"][8], layer["router"][1]) and np.array_equal(re["gate_exps"][9], layer["gate_exps"][5])


def test_owner_ranges_and_split_sizes():
    assert ep.owner_ranges(512, 8)[3] == (192, 64)
    with pytest.raises(ValueError):
        ep.owner_ranges(512, 3)
    cnt_all = np.array([[1, 2, 3, 4], [5, 6, 7, 8]], dtype=np.int32)  # two ranks, four experts
    assert ep.split_sizes(cnt_all, 0) == ([3, 7], [3, 11])
    assert ep.split_sizes(cnt_all, 1) == ([11, 15], [7, 15])
    assert list(ep.received_ids(cnt_all, 1)) == [2] * 3 + [3] * 4 + [2] * 7 + [3] * 8
