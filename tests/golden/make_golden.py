"""Writes the golden vectors under tests/golden/ from gguf-py (the `gguf` package, pinned by the reference in
pyproject.toml to the llama.cpp commit its ggml comes from): for each block format, seeded random blocks and gguf-py's
dequantisation of them; for q8_0, gguf-py's quantisation of a seeded row. Run once, here, where gguf-py is installed;
the .npz files are committed and the tests read only them.

    python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np
from gguf import quants

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", ".."))
from c0ven_b200 import synth  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))
CLASSES = {synth.Q8_0: quants.Q8_0, synth.Q4_K: quants.Q4_K, synth.Q6_K: quants.Q6_K, synth.IQ3_S: quants.IQ3_S,
           synth.IQ4_NL: quants.IQ4_NL, synth.IQ4_XS: quants.IQ4_XS, synth.IQ3_XXS: quants.IQ3_XXS, synth.IQ2_S: quants.IQ2_S}


def main():
    quants.IQ3_S.init_grid()
    rng = np.random.default_rng(20261125)
    out = {}
    for t, cls in CLASSES.items():
        blocks = synth.random_blocks(t, 24, rng)
        # Edge bytes: all-zero and all-ones quants in two of the blocks, scales kept.
        keep = blocks[:2].copy()
        blocks[0] = 0
        blocks[1] = 255
        if t == synth.Q6_K:
            blocks[:2, 208:210] = keep[:, 208:210]
        elif t == synth.Q4_K:
            blocks[:2, 0:4] = keep[:, 0:4]
        else:
            blocks[:2, 0:2] = keep[:, 0:2]
        out[f"blocks_{t}"] = blocks
        if hasattr(cls, "init_grid"):
            cls.init_grid()
        out[f"values_{t}"] = cls.dequantize_blocks(blocks).astype(np.float32).reshape(-1)
    x = (rng.standard_normal(32 * 40) * np.repeat(rng.uniform(0.01, 30, 40), 32)).astype(np.float32)
    x[:32] = 0.0  # a block of zeros: d = 0
    x[32:64] = np.round(x[32:64]) + 0.5  # ties
    out["q8_0_x"] = x
    out["q8_0_blocks"] = quants.Q8_0.quantize_blocks(x.reshape(-1, 32))
    np.savez_compressed(os.path.join(HERE, "gguf_py_vectors.npz"), **out)
    print("wrote", os.path.join(HERE, "gguf_py_vectors.npz"))


if __name__ == "__main__":
    main()
