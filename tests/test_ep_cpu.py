"""Expert parallel on two CPU ranks (gloo): the exchange logic of c0ven_b200.ep (split sizes, the two all-to-alls,
destination order, results back in place) with a CPU stand-in for the GPU stages. Each rank's outputs must be the
bits the oracle gives for that rank's rows on one process."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from c0ven_b200 import ep, synth


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, T, q):
    import sys
    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    from ep_common import OracleStages
    from oracle import oracle as O

    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        layer = synth.make_layer(n_embd=256, n_ff=256, n_experts=32, n_used=4, gate_type=synth.Q4_K, zipf_s=1.1, seed=3)
        x = synth.make_input(T[rank], 256, seed=10 + rank)
        moe = ep.ExpertParallelMoE(OracleStages(layer, rank, world))
        out = moe.forward(torch.from_numpy(x)).numpy()
        ref = O.moe_forward(layer, x)[0]
        q.put((rank, bool(np.array_equal(out, ref)), moe.sent_rows, moe.received_rows))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("T", [(37, 5), (1, 64)])
def test_two_ranks_give_the_single_process_bits(T):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, T, q)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    res = sorted(q.get(timeout=5) for _ in range(2))
    assert all(ok for _, ok, _, _ in res)
    # What one rank sent to the other is what the other received from it.
    assert res[0][2] == res[1][3] and res[1][2] == res[0][3]


def test_owner_ranges_and_split_sizes():
    assert ep.owner_ranges(512, 8)[3] == (192, 64)
    with pytest.raises(ValueError):
        ep.owner_ranges(512, 3)
    cnt_all = np.array([[1, 2, 3, 4], [5, 6, 7, 8]], dtype=np.int32)  # two ranks, four experts
    assert ep.split_sizes(cnt_all, 0) == ([3, 7], [3, 11])
    assert ep.split_sizes(cnt_all, 1) == ([11, 15], [7, 15])
    assert list(ep.received_ids(cnt_all, 1)) == [2] * 3 + [3] * 4 + [2] * 7 + [3] * 8
