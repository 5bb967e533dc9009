"""Seeded synthetic weights and inputs for the MoE layer, in the GGUF block formats of shared/quant.h.

The value distributions are the ones the benchmark configurations state: Q8_0 int8 codes uniform in [-127, 127] with
f16 d ~ U(1e-4, 3e-4); Q4_K nibbles uniform, 6-bit scales and minimums uniform, f16 d and dmin ~ U(1e-4, 1e-3);
Q6_K codes uniform, int8 sub-scales uniform, f16 d ~ U(2e-5, 2e-4) (chosen so its weights are about the size of
Q4_K's); IQ3_S grid indices, signs and 4-bit scales uniform, f16 d ~ U(1e-4, 1e-3). In spirit this is the reference's
test::random_blocks (core/tests/test_util.h:62-103): random bytes, then scales set so the weights stay small.
"""
from __future__ import annotations

import numpy as np

Q8_0, Q4_K, Q6_K, IQ3_XXS, IQ4_NL, IQ3_S, IQ2_S, IQ4_XS, Q2_0 = 8, 12, 14, 18, 20, 21, 22, 23, 42
BLOCK_VALUES = {Q8_0: 32, Q4_K: 256, Q6_K: 256, IQ3_S: 256, IQ4_NL: 32, IQ4_XS: 256, IQ3_XXS: 256, IQ2_S: 256, Q2_0: 64}
BLOCK_BYTES = {Q8_0: 34, Q4_K: 144, Q6_K: 210, IQ3_S: 110, IQ4_NL: 18, IQ4_XS: 136, IQ3_XXS: 98, IQ2_S: 82, Q2_0: 18}
TYPE_NAMES = {Q8_0: "Q8_0", Q4_K: "Q4_K", Q6_K: "Q6_K", IQ3_S: "IQ3_S", IQ4_NL: "IQ4_NL", IQ4_XS: "IQ4_XS", IQ3_XXS: "IQ3_XXS", IQ2_S: "IQ2_S", Q2_0: "Q2_0"}
TYPE_IDS = {v: k for k, v in TYPE_NAMES.items()}


def row_bytes(t: int, n: int) -> int:
    return n // BLOCK_VALUES[t] * BLOCK_BYTES[t]


def _f16_bytes(rng, n, lo, hi):
    return rng.uniform(lo, hi, size=n).astype(np.float16).view(np.uint8).reshape(n, 2)


def random_blocks(t: int, nblocks: int, rng: np.random.Generator) -> np.ndarray:
    """nblocks blocks of type t in the file's layout, as a uint8 array [nblocks, block bytes]."""
    b = rng.integers(0, 256, size=(nblocks, BLOCK_BYTES[t]), dtype=np.uint8)
    if t == Q8_0:
        q = b[:, 2:].view(np.int8)
        q[q == -128] = -127
        b[:, 0:2] = _f16_bytes(rng, nblocks, 1e-4, 3e-4)
    elif t == Q4_K:
        b[:, 0:2] = _f16_bytes(rng, nblocks, 1e-4, 1e-3)
        b[:, 2:4] = _f16_bytes(rng, nblocks, 1e-4, 1e-3)
    elif t == Q6_K:
        b[:, 208:210] = _f16_bytes(rng, nblocks, 2e-5, 2e-4)
    elif t == IQ3_S:
        b[:, 0:2] = _f16_bytes(rng, nblocks, 1e-4, 1e-3)
    elif t == IQ3_XXS:  # codebook bytes 4 .. 62 times (0.5 + s) / 2: about IQ3_S's size
        b[:, 0:2] = _f16_bytes(rng, nblocks, 1e-4, 1e-3)
    elif t == IQ2_S:    # codebook bytes 8, 25, 43 times (0.5 + s) / 4
        b[:, 0:2] = _f16_bytes(rng, nblocks, 2.5e-4, 2.5e-3)
    elif t == Q2_0:     # codes -1 .. 2 times d
        b[:, 0:2] = _f16_bytes(rng, nblocks, 5e-3, 2e-2)
    elif t == IQ4_NL:   # the table's values reach 127: scales as Q8_0's
        b[:, 0:2] = _f16_bytes(rng, nblocks, 1e-4, 3e-4)
    elif t == IQ4_XS:   # times a 6-bit scale minus 32: d chosen so that the weights are about the size of the others'
        b[:, 0:2] = _f16_bytes(rng, nblocks, 5e-6, 2e-5)
    else:
        raise ValueError(f"no generator for type {t}")
    return b


def random_matrix(t: int, rows: int, cols: int, rng) -> np.ndarray:
    """rows x cols values as uint8 [rows, row bytes]."""
    return random_blocks(t, rows * cols // BLOCK_VALUES[t], rng).reshape(rows, row_bytes(t, cols))


def zipf_bias(n_experts: int, s: float, rng) -> np.ndarray:
    """b_e = ln(p_rank(e)) with p_r proportional to r^-s over a seeded permutation of the experts, p_1 = 1."""
    rank = rng.permutation(n_experts) + 1
    return (-s * np.log(rank.astype(np.float64))).astype(np.float32)


def make_layer(n_embd=2048, n_ff=512, n_experts=512, n_used=10, gate_type=Q8_0, down_type=None,
               shexp_gate_type=None, shexp_down_type=None, zipf_s=0.0, seed=0, swiglu_limit=0.0) -> dict:
    """One layer's weights: router [NE][E] f32 ~ N(0, 0.02), the shared expert's gate vector [E] ~ N(0, 0.02), an
    optional per-expert router bias, and the experts' three matrices in the file's layout ([NE][rows][row bytes])."""
    down_type = gate_type if down_type is None else down_type
    shexp_gate_type = gate_type if shexp_gate_type is None else shexp_gate_type
    shexp_down_type = down_type if shexp_down_type is None else shexp_down_type
    rng = np.random.default_rng(seed)
    L = dict(n_embd=n_embd, n_ff=n_ff, n_experts=n_experts, n_used=n_used, gate_type=gate_type, down_type=down_type,
             shexp_gate_type=shexp_gate_type, shexp_down_type=shexp_down_type, swiglu_limit=swiglu_limit)
    L["router"] = (rng.standard_normal((n_experts, n_embd)) * 0.02).astype(np.float32)
    L["shexp_gate_inp"] = (rng.standard_normal(n_embd) * 0.02).astype(np.float32)
    L["router_bias"] = zipf_bias(n_experts, zipf_s, rng) if zipf_s > 0 else None
    gb, db = row_bytes(gate_type, n_embd), row_bytes(down_type, n_ff)
    L["gate_exps"] = random_matrix(gate_type, n_experts * n_ff, n_embd, rng).reshape(n_experts, n_ff, gb)
    L["up_exps"] = random_matrix(gate_type, n_experts * n_ff, n_embd, rng).reshape(n_experts, n_ff, gb)
    L["down_exps"] = random_matrix(down_type, n_experts * n_embd, n_ff, rng).reshape(n_experts, n_embd, db)
    L["gate_shexp"] = random_matrix(shexp_gate_type, n_ff, n_embd, rng)
    L["up_shexp"] = random_matrix(shexp_gate_type, n_ff, n_embd, rng)
    L["down_shexp"] = random_matrix(shexp_down_type, n_embd, n_ff, rng)
    return L


def make_input(T: int, n_embd: int, seed=1) -> np.ndarray:
    """Activations ~ N(0, 1), f32 [T][E]."""
    return np.random.default_rng(seed).standard_normal((T, n_embd)).astype(np.float32)


# The benchmark configurations (hidden 2048, expert FFN 512, 512 experts, top 10, one shared expert).
CONFIGS = {
    "decode1_q8_0": dict(tokens=1, runs=[1], gate_type=Q8_0, zipf_s=0.0),
    "ragged3521_q4_k_zipf": dict(tokens=3521, runs=[1, 8, 512, 3000], gate_type=Q4_K, zipf_s=1.1),
    "stack48_verify32_iq3_s": dict(tokens=32, runs=[8, 8, 8, 8], gate_type=IQ3_S, zipf_s=0.0, layers=48, scaling="strong"),
    "prefill32768_q4_k": dict(tokens=32768, runs=[32768], gate_type=Q4_K, zipf_s=0.0, scaling="strong"),
    "sweep_q4k_q6k_q8_0": dict(tokens=[1, 4, 32, 256, 2048, 8192], gate_type=Q4_K, down_type=Q6_K,
                               shexp_gate_type=Q8_0, shexp_down_type=Q8_0, zipf_s=1.1),
}


def expert_bytes(gate_type: int, down_type: int, n_embd=2048, n_ff=512) -> int:
    """Bytes of one expert's three matrices."""
    return 2 * n_ff * row_bytes(gate_type, n_embd) + n_embd * row_bytes(down_type, n_ff)


def write_gguf(path: str, layers: list, arch: str = "qwen4exp", router_type: str = "f32", token_embd=None, ffn_norms=None,
               output_norm=None, output=None) -> None:
    """Writes layers (dicts as make_layer returns) as a GGUF version 3 file with the reference's tensor names
    (blk.N.ffn_gate_inp.weight, ffn_gate_inp_shexp.weight, ffn_{gate,up,down}_exps.weight, ffn_{gate,up,down}_shexp.weight:
    docs/spec/MODEL_LAYER.md 4.1) and the metadata a reader needs (block_count, expert_count, expert_used_count,
    embedding_length, expert_feed_forward_length). Needs gguf-py. router_type: "f32", "f16" or "bf16". For a whole model
    (what engine_open reads): token_embd [vocab][n_embd] f32, and optionally ffn_norms (one [n_embd] vector a layer, as
    blk.N.ffn_norm.weight), output_norm [n_embd] and output [vocab][n_embd] (absent: the embedding is tied)."""
    import gguf

    w = gguf.GGUFWriter(str(path), arch)
    L0 = layers[0]
    w.add_block_count(len(layers))
    w.add_embedding_length(L0["n_embd"])
    w.add_expert_count(L0["n_experts"])
    w.add_expert_used_count(L0["n_used"])
    w.add_expert_feed_forward_length(L0["n_ff"])
    qt = gguf.GGMLQuantizationType

    def plain(a):
        a = np.ascontiguousarray(a, dtype=np.float32)
        if router_type == "f16":
            return a.astype(np.float16), None
        if router_type == "bf16":
            u = a.view(np.uint32)
            return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16).view(np.uint8).reshape(a.shape[:-1] + (a.shape[-1] * 2,)), qt.BF16
        return a, None

    if token_embd is not None:
        w.add_tensor("token_embd.weight", np.ascontiguousarray(token_embd, dtype=np.float32))
    if output_norm is not None:
        w.add_tensor("output_norm.weight", np.ascontiguousarray(output_norm, dtype=np.float32))
    if output is not None:
        w.add_tensor("output.weight", np.ascontiguousarray(output, dtype=np.float32))
    for i, L in enumerate(layers):
        if ffn_norms is not None:
            w.add_tensor(f"blk.{i}.ffn_norm.weight", np.ascontiguousarray(ffn_norms[i], dtype=np.float32))
        r, rt = plain(L["router"])
        w.add_tensor(f"blk.{i}.ffn_gate_inp.weight", r, raw_dtype=rt)
        for name, key, t in (("ffn_gate_exps", "gate_exps", L["gate_type"]), ("ffn_up_exps", "up_exps", L["gate_type"]),
                             ("ffn_down_exps", "down_exps", L["down_type"])):
            w.add_tensor(f"blk.{i}.{name}.weight", np.ascontiguousarray(L[key]), raw_dtype=qt(t))
        if L.get("gate_shexp") is not None:
            g, gt = plain(L["shexp_gate_inp"])
            w.add_tensor(f"blk.{i}.ffn_gate_inp_shexp.weight", g, raw_dtype=gt)
            for name, key, t in (("ffn_gate_shexp", "gate_shexp", L["shexp_gate_type"]), ("ffn_up_shexp", "up_shexp", L["shexp_gate_type"]),
                                 ("ffn_down_shexp", "down_shexp", L["shexp_down_type"])):
                w.add_tensor(f"blk.{i}.{name}.weight", np.ascontiguousarray(L[key]), raw_dtype=qt(t))
    w.write_header_to_file()
    w.write_kv_data_to_file()
    w.write_tensors_to_file()
    w.close()
