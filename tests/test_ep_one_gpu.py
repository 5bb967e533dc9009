"""The expert-parallel stage calls of the C ABI on ONE GPU: two layers, each holding half the experts, play the two
ranks one after the other, and the all-to-alls between them are plain tensor copies (no process group, no kernel waits
for another). A rank's outputs must equal, bit for bit, what a layer holding every expert gives for the same rows when
every expert takes the tile kernels on both sides and the results travel as f16, the form the one layer keeps them in
between its down kernel and its combine; and the ids the device derives from the gathered counts must be the host
function's."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _exchange(parts, sizes):
    """all_to_all_single by hand: parts[r] is rank r's send buffer, sizes[r][d] the rows it sends to rank d. Returns the
    receive buffers: for each destination the sources one after another."""
    import torch

    world = len(parts)
    offs = [np.concatenate([[0], np.cumsum(s)]) for s in sizes]
    return [torch.cat([parts[r][offs[r][d]:offs[r][d + 1]] for r in range(world)]) for d in range(world)]


@pytest.mark.parametrize("wtype,rows", [("Q4_K", (300, 41)), ("IQ3_S", (7, 1)), ("Q8_0", (64, 33))])
def test_two_ranges_on_one_gpu_match_the_whole_layer(wtype, rows):
    import torch

    from c0ven_b200 import MoELayer, ep, synth
    from oracle import oracle as O

    world = 2
    layer = synth.make_layer(n_embd=512, n_ff=256, n_experts=32, n_used=4, gate_type=synth.TYPE_IDS[wtype], zipf_s=1.1, seed=70)
    xs = [synth.make_input(rows[r], 512, seed=30 + r) for r in range(world)]
    single = MoELayer(layer, max_tokens=512, tensor_min_rows=1)
    want = [single.forward(x) for x in xs]
    single.close()
    stages = [ep.GpuStages(layer, r, world, max_tokens=512, device=0, y_f16=True, tensor_min_rows=1, profile=True) for r in range(world)]
    try:
        xd = [torch.from_numpy(x).cuda() for x in xs]
        cnts = [st.route(xd[r]) for r, st in enumerate(stages)]
        for st in stages:
            st.sync()
        cnt_all = torch.cat(cnts)
        torch.cuda.synchronize()
        counts = cnt_all.cpu().numpy().reshape(world, -1)
        splits = [ep.split_sizes(counts, r) for r in range(world)]
        sent = []
        for st in stages:
            rows_out = st.gather()
            st.sync()
            sent.append(rows_out.clone())
        rows_in = [t.contiguous() for t in _exchange(sent, [s[0] for s in splits])]
        torch.cuda.synchronize()  # the copies ran on torch's stream, the stages run on the layers' own
        ys = []
        for r, st in enumerate(stages):
            R = sum(splits[r][1])
            assert rows_in[r].shape[0] == R
            ids_dev = st.ids_from_counts(cnt_all, world, R)
            st.sync()
            np.testing.assert_array_equal(ids_dev.cpu().numpy(), ep.received_ids(counts, r))
            y_in = st.experts(rows_in[r], ids_dev)
            st.sync()
            ys.append(y_in.clone())
            torch.cuda.synchronize()
        # Results go back the way the rows came: rank d returns to source r the rows r sent it.
        back = [t.contiguous() for t in _exchange(ys, [s[1] for s in splits])]
        torch.cuda.synchronize()
        for r, st in enumerate(stages):
            st.shared()
            out = torch.empty_like(xd[r])
            st.combine(back[r], out)
            st.sync()
            got = out.cpu().numpy()
            ref = O.moe_forward(layer, xs[r])[0]
            assert np.abs(got - ref).max() / np.abs(ref).max() <= 1e-2
            np.testing.assert_array_equal(got, want[r])
    finally:
        for st in stages:
            st.close()


@pytest.mark.parametrize("wtype,rows,world", [("Q4_K", (300, 41), 2), ("IQ3_S", (7, 1, 30, 12), 4), ("Q8_0", (64, 33), 2),
                                              ("Q4_K", (40, 3, 17, 1, 64, 9, 25, 12), 8)])
def test_one_row_per_token_and_gpu_on_one_gpu(wtype, rows, world):
    """The same on one GPU for the other form of the exchange: one row per (token, GPU) out, one weighted partial sum
    back. Each rank's outputs are held to the oracle (and so to the whole layer's) within the layer's bar; the rows
    that cross are counted against the plan's totals; the lists that travel with them name only the receiver's experts."""
    import torch

    from c0ven_b200 import ep, synth
    from oracle import oracle as O

    K = 4
    layer = synth.make_layer(n_embd=512, n_ff=256, n_experts=32, n_used=K, gate_type=synth.TYPE_IDS[wtype], zipf_s=1.1, seed=71)
    xs = [synth.make_input(rows[r], 512, seed=40 + r) for r in range(world)]
    stages = [ep.GpuStages(layer, r, world, max_tokens=512, device=0, tensor_min_rows=1, profile=True) for r in range(world)]
    try:
        xd = [torch.from_numpy(x).cuda() for x in xs]
        tots = []
        for r, st in enumerate(stages):
            st.route(xd[r])
            tots.append(st.plan())
            st.sync()
        m = torch.stack(tots).cpu().numpy().reshape(world, 2, 8)
        for r, st in enumerate(stages):   # the plan against the routing it came from
            ids = st.moe.route(rows[r])[0]
            owner = ids // (32 // world)
            assert [int(v) for v in m[r, 0, :world]] == [int((owner == g).any(1).sum()) for g in range(world)]
            assert [int(v) for v in m[r, 1, :world]] == [int((owner == g).sum()) for g in range(world)]
        sent = []
        for r, st in enumerate(stages):
            d = st.dispatch(int(m[r, 0, :world].sum()))
            st.sync()
            sent.append(d.clone())
        assert sum(s.shape[0] for s in sent) < sum(rows) * K or world == 1
        rows_in = [t.contiguous() for t in _exchange(sent, [[int(v) for v in m[r, 0, :world]] for r in range(world)])]
        torch.cuda.synchronize()
        ys = []
        for r, st in enumerate(stages):
            wb = st.moe.wire_row_bytes
            meta = rows_in[r][:, wb:wb + 32].cpu().numpy().view(np.uint16)[:, :K]
            assert np.all((meta == 0xFFFF) | (meta < 32 // world)) and int((meta != 0xFFFF).sum()) == int(m[:, 1, r].sum())
            y = st.experts_partial(rows_in[r], int(m[:, 1, r].sum()))
            st.sync()
            ys.append(y.clone())
            torch.cuda.synchronize()
        back = [t.contiguous() for t in _exchange(ys, [[int(v) for v in m[:, 0, r]] for r in range(world)])]
        torch.cuda.synchronize()
        for r, st in enumerate(stages):
            st.shared()
            out = torch.empty_like(xd[r])
            st.combine_partials(back[r], out)
            st.sync()
            got = out.cpu().numpy()
            ref = O.moe_forward(layer, xs[r])[0]
            assert np.abs(got - ref).max() / np.abs(ref).max() <= 1e-2
    finally:
        for st in stages:
            st.close()
