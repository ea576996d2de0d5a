"""Synthetic checkpoints with the tensor names, shapes, dtypes and file counts of the benchmark
configurations, plus the tensor-parallel plan (which dimension each tensor is split on).

No real model weights are involved.  Values come from one seeded pool per dtype (normal or
uniform, as the configuration states) from which every tensor takes a window at its own
offset, so files are written at memory-copy speed, every tensor has distinct content, and any
process can regenerate the exact bytes of any tensor from (seed, tensor index).

``python -m tests.synth <config> <out_dir> [--scale tiny]`` (from the repository root) writes a checkpoint.
"""

from __future__ import annotations

import json
import os
import struct
from dataclasses import dataclass
from typing import Dict, Iterator, List, Optional, Sequence, Tuple

import numpy as np

# action of the TP plan for a tensor: ("shard", dim) | ("replicate",) | ("push", dst_rank)
Action = Tuple


@dataclass
class TensorSpec:
    name: str
    dtype: str            # safetensors dtype string: "BF16", "F16", "F32", ...
    shape: Tuple[int, ...]
    action: Action

    @property
    def nbytes(self) -> int:
        n = _ITEMSIZE[self.dtype]
        for s in self.shape:
            n *= s
        return n


@dataclass
class CheckpointSpec:
    name: str
    tensors: List[TensorSpec]
    n_files: int
    seed: int
    dist: str = "normal"          # "normal" -> N(0, 0.02), "uniform" -> U(-1, 1)
    odd_header: bool = False      # pad the JSON so that 8 + len(JSON) is odd
    tp: int = 8                   # tensor-parallel degree the configuration is quoted on
    note: str = ""

    @property
    def data_bytes(self) -> int:
        return sum(t.nbytes for t in self.tensors)


_ITEMSIZE = {"BF16": 2, "F16": 2, "F32": 4, "F64": 8, "I8": 1, "U8": 1, "I32": 4, "I64": 8}


# ------------------------------------------------------------------------------------------
# architectures
# ------------------------------------------------------------------------------------------
def llama(name: str, hidden: int, layers: int, q_heads: int, kv_heads: int, head_dim: int, ffn: int,
          vocab: int, dtype: str, norm_dtype: str, n_files: int, seed: int, tp: int,
          dist: str = "normal", odd_header: bool = False) -> CheckpointSpec:
    """Llama-shaped checkpoint: q/k/v/gate/up and the vocabulary matrices split on dim 0,
    o_proj/down_proj on dim 1, norms replicated."""
    t: List[TensorSpec] = [TensorSpec("model.embed_tokens.weight", dtype, (vocab, hidden), ("shard", 0))]
    for i in range(layers):
        p = f"model.layers.{i}."
        t += [
            TensorSpec(p + "input_layernorm.weight", norm_dtype, (hidden,), ("replicate",)),
            TensorSpec(p + "self_attn.q_proj.weight", dtype, (q_heads * head_dim, hidden), ("shard", 0)),
            TensorSpec(p + "self_attn.k_proj.weight", dtype, (kv_heads * head_dim, hidden), ("shard", 0)),
            TensorSpec(p + "self_attn.v_proj.weight", dtype, (kv_heads * head_dim, hidden), ("shard", 0)),
            TensorSpec(p + "self_attn.o_proj.weight", dtype, (hidden, q_heads * head_dim), ("shard", 1)),
            TensorSpec(p + "post_attention_layernorm.weight", norm_dtype, (hidden,), ("replicate",)),
            TensorSpec(p + "mlp.gate_proj.weight", dtype, (ffn, hidden), ("shard", 0)),
            TensorSpec(p + "mlp.up_proj.weight", dtype, (ffn, hidden), ("shard", 0)),
            TensorSpec(p + "mlp.down_proj.weight", dtype, (hidden, ffn), ("shard", 1)),
        ]
    t += [
        TensorSpec("model.norm.weight", norm_dtype, (hidden,), ("replicate",)),
        TensorSpec("lm_head.weight", dtype, (vocab, hidden), ("shard", 0)),
    ]
    return CheckpointSpec(name, t, n_files, seed, dist, odd_header, tp)


def gpt2(name: str, hidden: int, layers: int, vocab: int, positions: int, seed: int) -> CheckpointSpec:
    """GPT-2-shaped single file, fp16, loaded whole (world size 1)."""
    d = "F16"
    t: List[TensorSpec] = [
        TensorSpec("wte.weight", d, (vocab, hidden), ("replicate",)),
        TensorSpec("wpe.weight", d, (positions, hidden), ("replicate",)),
    ]
    for i in range(layers):
        p = f"h.{i}."
        t += [
            TensorSpec(p + "ln_1.weight", d, (hidden,), ("replicate",)),
            TensorSpec(p + "ln_1.bias", d, (hidden,), ("replicate",)),
            TensorSpec(p + "attn.c_attn.weight", d, (hidden, 3 * hidden), ("shard", 1)),
            TensorSpec(p + "attn.c_attn.bias", d, (3 * hidden,), ("shard", 0)),
            TensorSpec(p + "attn.c_proj.weight", d, (hidden, hidden), ("shard", 0)),
            TensorSpec(p + "attn.c_proj.bias", d, (hidden,), ("replicate",)),
            TensorSpec(p + "ln_2.weight", d, (hidden,), ("replicate",)),
            TensorSpec(p + "ln_2.bias", d, (hidden,), ("replicate",)),
            TensorSpec(p + "mlp.c_fc.weight", d, (hidden, 4 * hidden), ("shard", 1)),
            TensorSpec(p + "mlp.c_fc.bias", d, (4 * hidden,), ("shard", 0)),
            TensorSpec(p + "mlp.c_proj.weight", d, (4 * hidden, hidden), ("shard", 0)),
            TensorSpec(p + "mlp.c_proj.bias", d, (hidden,), ("replicate",)),
        ]
    t += [TensorSpec("ln_f.weight", d, (hidden,), ("replicate",)),
          TensorSpec("ln_f.bias", d, (hidden,), ("replicate",))]
    return CheckpointSpec(name, t, 1, seed, "normal", False, 1)


def mixtral(name: str, hidden: int, layers: int, experts: int, q_heads: int, kv_heads: int,
            head_dim: int, ffn: int, vocab: int, n_files: int, seed: int, tp: int) -> CheckpointSpec:
    """Mixtral-shaped checkpoint: expert e goes whole to rank e (push), attention is TP-sharded,
    router and norms are replicated."""
    d = "BF16"
    t: List[TensorSpec] = [TensorSpec("model.embed_tokens.weight", d, (vocab, hidden), ("shard", 0))]
    for i in range(layers):
        p = f"model.layers.{i}."
        t += [
            TensorSpec(p + "input_layernorm.weight", d, (hidden,), ("replicate",)),
            TensorSpec(p + "self_attn.q_proj.weight", d, (q_heads * head_dim, hidden), ("shard", 0)),
            TensorSpec(p + "self_attn.k_proj.weight", d, (kv_heads * head_dim, hidden), ("shard", 0)),
            TensorSpec(p + "self_attn.v_proj.weight", d, (kv_heads * head_dim, hidden), ("shard", 0)),
            TensorSpec(p + "self_attn.o_proj.weight", d, (hidden, q_heads * head_dim), ("shard", 1)),
            TensorSpec(p + "post_attention_layernorm.weight", d, (hidden,), ("replicate",)),
            TensorSpec(p + "block_sparse_moe.gate.weight", d, (experts, hidden), ("replicate",)),
        ]
        for e in range(experts):
            q = p + f"block_sparse_moe.experts.{e}."
            t += [
                TensorSpec(q + "w1.weight", d, (ffn, hidden), ("push", e)),
                TensorSpec(q + "w2.weight", d, (hidden, ffn), ("push", e)),
                TensorSpec(q + "w3.weight", d, (ffn, hidden), ("push", e)),
            ]
    t += [TensorSpec("model.norm.weight", d, (hidden,), ("replicate",)),
          TensorSpec("lm_head.weight", d, (vocab, hidden), ("shard", 0))]
    return CheckpointSpec(name, t, n_files, seed, "normal", False, tp)


def config(name: str, scale: str = "full") -> CheckpointSpec:
    """The five benchmark configurations; ``scale="tiny"`` gives a twin with the same tensor
    names, dtypes, split dimensions and file count but small extents (for tests)."""
    tiny = scale == "tiny"
    if name == "gpt2-small":
        return gpt2(name, 48 if tiny else 768, 2 if tiny else 12, 1031 if tiny else 50257,
                    64 if tiny else 1024, seed=0)
    if name == "llama3-8b":
        if tiny:
            return llama(name, 128, 4, 8, 8, 16, 448, 1024, "BF16", "BF16", 4, 1, 8)
        return llama(name, 4096, 32, 32, 8, 128, 14336, 128256, "BF16", "BF16", 4, 1, 8)
    if name == "llama2-13b":
        if tiny:
            return llama(name, 160, 3, 8, 8, 20, 432, 1000, "F16", "F32", 3, 2, 4, "uniform", True)
        return llama(name, 5120, 40, 40, 40, 128, 13824, 32000, "F16", "F32", 3, 2, 4, "uniform", True)
    if name == "llama3-70b":
        if tiny:
            return llama(name, 256, 6, 16, 8, 16, 896, 2048, "BF16", "BF16", 30, 3, 8)
        return llama(name, 8192, 80, 64, 8, 128, 28672, 128256, "BF16", "BF16", 30, 3, 8)
    if name == "mixtral-8x7b":
        if tiny:
            return mixtral(name, 128, 3, 8, 8, 8, 16, 448, 1000, 19, 4, 8)
        return mixtral(name, 4096, 32, 8, 32, 8, 128, 14336, 32000, 19, 4, 8)
    raise KeyError(f"unknown configuration {name!r}")


CONFIG_NAMES = ("gpt2-small", "llama3-8b", "llama2-13b", "llama3-70b", "mixtral-8x7b")


# ------------------------------------------------------------------------------------------
# values
# ------------------------------------------------------------------------------------------
_POOL_ELEMS = 1 << 22  # elements per pool (8 MiB of 16-bit values)
_NP_VIEW = {"BF16": np.uint16, "F16": np.float16, "F32": np.float32, "F64": np.float64,
            "I8": np.int8, "U8": np.uint8, "I32": np.int32, "I64": np.int64}


def _pool(dtype: str, seed: int, dist: str) -> np.ndarray:
    """Seeded value pool of one dtype, returned as raw bytes (uint8)."""
    rng = np.random.default_rng([seed, sum(dtype.encode())])
    if dist == "uniform":
        x = rng.uniform(-1.0, 1.0, _POOL_ELEMS).astype(np.float32)
    else:
        x = (rng.standard_normal(_POOL_ELEMS, dtype=np.float32) * np.float32(0.02))
    if dtype == "BF16":
        # round-to-nearest-even truncation of fp32 to its upper 16 bits
        u = x.view(np.uint32)
        u = (u + np.uint32(0x7FFF) + ((u >> np.uint32(16)) & np.uint32(1))) >> np.uint32(16)
        out = u.astype(np.uint16)
    elif dtype in ("F16", "F32", "F64"):
        out = x.astype(_NP_VIEW[dtype])
    else:
        info = np.iinfo(_NP_VIEW[dtype])
        out = rng.integers(info.min, int(info.max) + 1, _POOL_ELEMS, dtype=_NP_VIEW[dtype])
    return out.view(np.uint8)


class ValueSource:
    """Bytes of tensor number ``index`` of a checkpoint: a window of the dtype's pool that
    starts at an offset derived from (seed, index) and wraps around."""

    def __init__(self, seed: int, dist: str):
        self.seed, self.dist = seed, dist
        self._pools: Dict[str, np.ndarray] = {}

    def pool(self, dtype: str) -> np.ndarray:
        if dtype not in self._pools:
            self._pools[dtype] = _pool(dtype, self.seed, self.dist)
        return self._pools[dtype]

    def chunks(self, dtype: str, index: int, nbytes: int) -> Iterator[np.ndarray]:
        pool = self.pool(dtype)
        item = _ITEMSIZE[dtype]
        start = ((index * 2654435761 + self.seed * 40503) % _POOL_ELEMS) * item
        left = nbytes
        while left > 0:
            take = min(left, pool.size - start)
            yield pool[start:start + take]
            left -= take
            start = 0

    def tensor_bytes(self, dtype: str, index: int, nbytes: int) -> np.ndarray:
        return np.concatenate(list(self.chunks(dtype, index, nbytes))) if nbytes else np.empty(0, np.uint8)


# ------------------------------------------------------------------------------------------
# files
# ------------------------------------------------------------------------------------------
def partition(spec: CheckpointSpec) -> List[List[int]]:
    """Tensor indices per file: consecutive runs of about equal bytes, never an empty file."""
    n = len(spec.tensors)
    files = min(spec.n_files, n)
    total = spec.data_bytes
    out: List[List[int]] = [[] for _ in range(files)]
    acc = 0
    f = 0
    for i, t in enumerate(spec.tensors):
        remaining_tensors = n - i
        remaining_files = files - f
        if out[f] and (acc >= total * (f + 1) / files or remaining_tensors <= remaining_files - 1):
            f = min(f + 1, files - 1)
        out[f].append(i)
        acc += t.nbytes
    return [g for g in out if g]


def header_bytes(entries: "Dict[str, dict]", odd: bool, metadata: Optional[Dict[str, str]] = None) -> bytes:
    """8-byte little-endian length + JSON, space padded so that the data section starts on an
    8-byte boundary (what ``safetensors`` writers do) or, with ``odd``, on an odd offset."""
    doc = dict(entries)
    if metadata:
        doc = {"__metadata__": metadata, **doc}
    body = json.dumps(doc, separators=(",", ":")).encode()
    pad = (-(8 + len(body))) % 8
    if odd:
        pad += 1
    body += b" " * pad
    return struct.pack("<Q", len(body)) + body


def file_name(spec: CheckpointSpec, k: int, n: int) -> str:
    return f"{spec.name}-{k + 1:05d}-of-{n:05d}.safetensors"


def write_checkpoint(spec: CheckpointSpec, out_dir: str, fsync: bool = True,
                     only_files: Optional[Sequence[int]] = None) -> List[str]:
    """Write the checkpoint's files (skipping files that exist with the right size); with
    ``only_files`` just the files of those indices.  Returns the paths written or found."""
    os.makedirs(out_dir, exist_ok=True)
    src = ValueSource(spec.seed, spec.dist)
    groups = partition(spec)
    wanted = None if only_files is None else set(only_files)
    paths: List[str] = []
    for k, group in enumerate(groups):
        if wanted is not None and k not in wanted:
            continue
        entries: Dict[str, dict] = {}
        off = 0
        for i in group:
            t = spec.tensors[i]
            entries[t.name] = {"dtype": t.dtype, "shape": list(t.shape), "data_offsets": [off, off + t.nbytes]}
            off += t.nbytes
        head = header_bytes(entries, spec.odd_header, {"format": "pt", "config": spec.name})
        path = os.path.join(out_dir, file_name(spec, k, len(groups)))
        paths.append(path)
        if os.path.exists(path) and os.path.getsize(path) == len(head) + off:
            continue
        tmp = path + ".tmp"
        with open(tmp, "wb", buffering=0) as f:
            f.write(head)
            for i in group:
                t = spec.tensors[i]
                for chunk in src.chunks(t.dtype, i, t.nbytes):
                    f.write(chunk.data)
            if fsync:
                os.fsync(f.fileno())
        os.replace(tmp, path)
    return paths


def expected_bytes(spec: CheckpointSpec, index: int) -> np.ndarray:
    """The exact bytes tensor ``index`` has in the written files."""
    t = spec.tensors[index]
    return ValueSource(spec.seed, spec.dist).tensor_bytes(t.dtype, index, t.nbytes)


def owners(paths: Sequence[str], world_size: int) -> Dict[int, List[str]]:
    """Round-robin file ownership: file i (in sorted order) belongs to rank i mod W."""
    out: Dict[int, List[str]] = {r: [] for r in range(world_size)}
    for i, p in enumerate(sorted(paths)):
        out[i % world_size].append(p)
    return out


def drop_page_cache(paths: Sequence[str]) -> None:
    """Ask the kernel to forget the cached pages of these files (cold-read measurements)."""
    for p in paths:
        fd = os.open(p, os.O_RDONLY)
        try:
            os.fsync(fd)
            os.posix_fadvise(fd, 0, 0, os.POSIX_FADV_DONTNEED)
        finally:
            os.close(fd)


if __name__ == "__main__":
    import argparse

    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("config", choices=CONFIG_NAMES)
    ap.add_argument("out_dir")
    ap.add_argument("--scale", default="full", choices=("full", "tiny"))
    a = ap.parse_args()
    s = config(a.config, a.scale)
    files = write_checkpoint(s, a.out_dir)
    print(f"{s.name}: {len(s.tensors)} tensors, {s.data_bytes} data bytes, {len(files)} files in {a.out_dir}")
