"""The library's GGUF reader without a GPU: a small file written with gguf-py (the writer the reference pins to its
llama.cpp commit) is opened through the C ABI, and the tensor table it reports (names, types, shapes in ggml's order,
offsets, sizes) is the one gguf-py's own reader finds; the bytes at those offsets are the tensors' bytes."""
import numpy as np
import pytest

from c0ven_b200 import MoEError, synth
from c0ven_b200.layer import GgufFile

gguf = pytest.importorskip("gguf")


@pytest.fixture(scope="module")
def small_file(tmp_path_factory):
    layers = [synth.make_layer(n_embd=256, n_ff=256, n_experts=32, n_used=4, gate_type=synth.Q4_K, down_type=synth.Q6_K,
                               shexp_gate_type=synth.Q8_0, shexp_down_type=synth.IQ3_S, seed=500 + i) for i in range(2)]
    path = tmp_path_factory.mktemp("gguf") / "two_layers.gguf"
    synth.write_gguf(path, layers, router_type="bf16")
    return path, layers


def test_tensor_table_matches_gguf_pys_reader(small_file):
    path, layers = small_file
    f = GgufFile(path)
    assert f.layers == 2
    mine = f.tensors()
    theirs = gguf.GGUFReader(str(path))
    assert set(mine) == {t.name for t in theirs.tensors}
    raw = open(path, "rb").read()
    for t in theirs.tensors:
        ty, shape, offset, nbytes = mine[t.name]
        assert ty == int(t.tensor_type) and shape == tuple(int(d) for d in t.shape)
        assert offset == t.data_offset and nbytes == t.n_bytes
        assert raw[offset:offset + nbytes] == t.data.tobytes()
    ty, shape, offset, nbytes = mine["blk.1.ffn_down_exps.weight"]
    assert ty == synth.Q6_K and shape == (256, 256, 32)
    assert raw[offset:offset + nbytes] == layers[1]["down_exps"].tobytes()
    f.close()


def test_a_file_that_is_not_gguf_is_refused(tmp_path):
    p = tmp_path / "junk.gguf"
    p.write_bytes(b"GGUF" + bytes(40))
    with pytest.raises(MoEError) as e:
        GgufFile(p)
    assert "version" in str(e.value)
    with pytest.raises(MoEError):
        GgufFile(tmp_path / "absent.gguf")
