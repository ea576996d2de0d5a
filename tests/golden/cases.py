"""Parity cases shared by the golden generator (which runs upstream) and the tests (which run
the oracle and the CUDA path): which synthetic checkpoint, how many ranks, which requests."""

import os
from typing import Dict, List, Tuple

import numpy as np

from tests import synth


def owners(paths: List[str], world: int) -> Dict[int, List[str]]:
    return synth.owners(paths, world)


# crafted checkpoint: mixed dtypes, a 3-byte tensor first so that later tensors sit at odd
# offsets inside the data section, N-d tensors split on inner dimensions, a scalar
CRAFTED = [
    # (file, name, dtype, shape, action)
    (0, "u8_3", "U8", (3,), ("replicate",)),
    (0, "f16_a", "F16", (6, 10), ("shard", 1)),
    (0, "f32_3d", "F32", (4, 6, 8), ("shard", 1)),
    (0, "i64", "I64", (8,), ("shard", 0)),
    (1, "bool", "BOOL", (16, 4), ("shard", 0)),
    (1, "f8", "F8_E4M3", (8, 16), ("shard", 1)),
    (1, "bf16_3d", "BF16", (2, 4, 6), ("shard", 2)),
    (1, "scalar", "F32", (), ("replicate",)),
    (1, "i8_odd", "I8", (4, 5), ("shard", 0)),
    (1, "f64", "F64", (2, 2), ("shard", 1)),
]
_CRAFTED_ITEM = {"U8": 1, "F16": 2, "F32": 4, "I64": 8, "BOOL": 1, "F8_E4M3": 1, "BF16": 2, "I8": 1,
                 "F64": 8}


def _write_crafted(out_dir: str) -> List[str]:
    os.makedirs(out_dir, exist_ok=True)
    rng = np.random.default_rng(1234)
    paths = []
    for f in (0, 1):
        entries, blobs, off = {}, [], 0
        for (ff, name, dtype, shape, _) in CRAFTED:
            if ff != f:
                continue
            n = _CRAFTED_ITEM[dtype] * int(np.prod(shape, dtype=np.int64))
            raw = rng.integers(0, 2 if dtype == "BOOL" else 256, n, dtype=np.uint8)
            if dtype in ("F16", "BF16", "F32", "F64", "F8_E4M3"):
                # keep clear of NaN bit patterns: they compare unequal in value-based checks
                raw = rng.integers(0, 120, n, dtype=np.uint8)
            entries[name] = {"dtype": dtype, "shape": list(shape), "data_offsets": [off, off + n]}
            blobs.append(raw.tobytes())
            off += n
        path = os.path.join(out_dir, f"crafted-{f}.safetensors")
        with open(path, "wb") as fh:
            fh.write(synth.header_bytes(entries, odd=(f == 1)))
            fh.write(b"".join(blobs))
            if f == 1:
                fh.write(b"\0" * 5)  # trailing padding after the last tensor is legal
        paths.append(path)
    return paths


def materialize(case: dict, out_dir: str) -> List[str]:
    """Write the case's checkpoint files (deterministic) and return their paths."""
    if case["config"] == "crafted":
        return _write_crafted(out_dir)
    return synth.write_checkpoint(synth.config(case["config"], "tiny"), out_dir, fsync=False)


def plan(case: dict) -> List[Tuple[str, tuple]]:
    """(tensor name, action) in request order; every rank issues them in this order."""
    if case["config"] == "crafted":
        skip = case.get("skip", ())
        return [(name, action) for (_, name, _, _, action) in CRAFTED if name not in skip]
    return [(t.name, t.action) for t in synth.config(case["config"], "tiny").tensors]


_L = "model.layers.1."
CASES = [
    {"id": "gpt2_w1", "config": "gpt2-small", "world": 1, "steps": [("plan",)]},
    {"id": "llama3_8b_w8", "config": "llama3-8b", "world": 8, "steps": [("plan",)]},
    {"id": "llama3_8b_w2_cols", "config": "llama3-8b", "world": 2, "steps": [
        ("multi_cols", "qkv", [_L + "self_attn.q_proj.weight", _L + "self_attn.k_proj.weight",
                               _L + "self_attn.v_proj.weight"], 0),
        ("multi_cols", "gate_up", [_L + "mlp.gate_proj.weight", "model.layers.3.mlp.up_proj.weight"], 0),
        ("multi_cols", "o_q_dim1", [_L + "self_attn.o_proj.weight", _L + "self_attn.q_proj.weight"], 1),
        ("as_dict", [("model.norm.weight", -1), ("lm_head.weight", 0),
                     ("model.layers.0.mlp.down_proj.weight", 1)]),
    ]},
    {"id": "llama2_13b_w4", "config": "llama2-13b", "world": 4, "steps": [("plan",)]},
    {"id": "llama2_13b_w1_gds", "config": "llama2-13b", "world": 1, "nogds": False, "steps": [("plan",)]},
    {"id": "llama3_70b_w8", "config": "llama3-70b", "world": 8, "steps": [("plan",)]},
    {"id": "mixtral_w8", "config": "mixtral-8x7b", "world": 8, "steps": [("plan",)]},
    {"id": "crafted_w1", "config": "crafted", "world": 1, "steps": [
        ("plan",), ("multi_cols", "cols_w1", ["f16_a", "f16_a"], 1)]},
    # upstream cannot scatter FP8 over gloo ("Invalid scalar type"), so f8 is left out here
    {"id": "crafted_w2", "config": "crafted", "world": 2, "skip": ("f8",), "steps": [("plan",)]},
]

# (shape, index expression) pairs for TensorFrame.__getitem__
FRAME_INDEXES = [
    ((10, 6), "slice(None)"), ((10, 6), "slice(2, 8)"), ((10, 6), "slice(8, 2, -1)"),
    ((10, 6), "slice(None, None, -2)"), ((10, 6), "slice(-3, None)"), ((10, 6), "slice(0, 100, 3)"),
    ((10, 6), "slice(5, 5)"), ((10, 6), "slice(7, 2)"), ((10, 6), "3"), ((10, 6), "-1"),
    ((10, 6), "10"), ((10, 6), "-11"), ((10, 6), "(slice(1, -1), slice(None, None, 2))"),
    ((10, 6), "(2, slice(1, 4))"), ((10, 6), "(slice(None), 5)"), ((4, 5, 6), "(slice(None), slice(1, 3))"),
    ((4, 5, 6), "(1, 2, 3)"), ((4, 5, 6), "(slice(None), slice(None), slice(4, 0, -2))"),
    ((7,), "slice(0, 7, 0)"), ((7,), "slice(-100, 100)"), ((0, 4), "slice(None)"),
]
