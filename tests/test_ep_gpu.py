"""Expert parallel on two B200s (NCCL): each rank holds half the experts; a rank's outputs must equal, bit for bit,
what one GPU holding every expert gives for the same rows when every expert takes the tile kernels on both
(tensor_min_rows 1) and the results travel as f16, the form one GPU keeps them in between its down kernel and its
combine; and stay within the layer's bar when they travel as f32. Needs two GPUs; skipped otherwise."""
import datetime
import os
import sys

import numpy as np
import pytest

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from ep_common import run_ranks  # noqa: E402

pytestmark = pytest.mark.gpu


def _worker(rank, world, port, q):
    import torch
    import torch.distributed as dist

    from c0ven_b200 import MoELayer, ep, synth
    from oracle import oracle as O

    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank),
                            timeout=datetime.timedelta(seconds=60))  # a lost peer ends the wait with an error
    res = []
    try:
        for t, T in ((synth.Q4_K, (300, 41)), (synth.IQ3_S, (7, 1))):
            layer = synth.make_layer(n_embd=512, n_ff=256, n_experts=32, n_used=4, gate_type=t, zipf_s=1.1, seed=50 + t)
            x = synth.make_input(T[rank], 512, seed=20 + rank)
            single = MoELayer(layer, max_tokens=512, device=rank, tensor_min_rows=1)
            want = single.forward(x)
            ids1 = single.route(T[rank])[0]
            single.close()
            ref = O.moe_forward(layer, x)[0]
            for f16 in (False, True):
                st = ep.GpuStages(layer, rank, world, max_tokens=512, device=rank, y_f16=f16, tensor_min_rows=1)
                moe = ep.ExpertParallelMoE(st, by_token=False)
                xd = torch.from_numpy(x).cuda()
                for _ in range(2):
                    out = moe.forward(xd)
                st.sync()
                got = out.cpu().numpy()
                rel = float(np.abs(got - ref).max() / np.abs(ref).max())
                res.append((t, f16, bool(np.array_equal(got, want)), rel, moe.sent_rows))
                st.close()
            # One row per (token, GPU), with the experts interleaved over the ranks: within the layer's bar of the oracle.
            st = ep.GpuStages(layer, rank, world, max_tokens=512, device=rank, tensor_min_rows=1, interleave=True)
            moe = ep.ExpertParallelMoE(st)
            for _ in range(2):
                out = moe.forward(torch.from_numpy(x).cuda())
            st.sync()
            got = out.cpu().numpy()
            res.append((t, "by_token", True, float(np.abs(got - ref).max() / np.abs(ref).max()), moe.sent_rows))
            # The host-buffer call, the step cut into three whose copies run beside their neighbours: the same bits
            # (every expert on the tile kernels, whose results for a row do not depend on the rows beside it).
            if min(T) >= 3:
                xh, oh = torch.from_numpy(x).pin_memory(), torch.empty((T[rank], 512), dtype=torch.float32).pin_memory()
                for _ in range(2):
                    moe.forward_host(xh, oh, chunks=3)
                res.append((t, "host", bool(np.array_equal(oh.numpy(), got)), float(np.abs(oh.numpy() - ref).max() / np.abs(ref).max()), moe.sent_rows))
                del xh, oh
            st.close()
        q.put((rank, res))
    finally:
        dist.destroy_process_group()


def test_two_gpus_match_one():
    import torch

    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    for rank, res in run_ranks(_worker, 2, timeout=600):
        for t, f16, same_bits, rel, sent in res:
            assert rel <= 1e-2, (rank, t, f16, rel)
            if f16 is True or f16 == "host":
                assert same_bits, (rank, t, f16)
            assert sent > 0
