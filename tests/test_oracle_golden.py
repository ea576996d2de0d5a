"""Pins the oracle (oracle/st_oracle.py) to outputs of upstream fastsafetensors itself.

tests/golden/reference_outputs.json was produced by running upstream on the same deterministic
tiny checkpoints (tests/golden/make_golden.py).  Every tensor every rank received there must
have the shape and bytes the oracle computes."""

import os
import sys

import pytest

from tests.golden import cases
from tests.helpers import digest_bytes

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from oracle import st_oracle  # noqa: E402


def _oracles(paths):
    by_name = {}
    for p in paths:
        fo = st_oracle.FileOracle(p)
        for n in fo.tensors:
            by_name[n] = fo
    return by_name


def expected_for_rank(case, paths, rank):
    """What the oracle says rank ``rank`` receives, keyed like the golden file."""
    world = case["world"]
    by_name = _oracles(paths)
    out = {}
    for step in case["steps"]:
        if step[0] == "plan":
            for name, action in cases.plan(case):
                fo = by_name[name]
                if action[0] == "shard":
                    raw, shape = fo.get_sharded(name, action[1], rank, world)
                elif action[0] == "replicate":
                    raw, shape = fo.get_tensor(name)
                else:
                    if world > 1 and action[1] % world != rank:
                        out[name] = None
                        continue
                    raw, shape = fo.get_tensor(name)
                out[name] = (shape, digest_bytes(raw))
        elif step[0] == "multi_cols":
            _, key, names, dim = step
            # groups by file in sorted (owner, file) order, names in given order inside a group
            order = sorted(paths)
            groups = {}
            for n in names:
                groups.setdefault(order.index(by_name[n].path), []).append(n)
            keyed = sorted(groups, key=lambda i: (i % world, i // world))
            parts = [by_name[groups[i][0]].get_multi_cols(groups[i], dim, rank, world) for i in keyed]
            if len(parts) == 1:
                raw, shape = parts[0]
            else:
                dtype = by_name[names[0]].tensors[names[0]]["dtype"]
                raw, shape = st_oracle.multi_cols([p[0] for p in parts], [p[1] for p in parts],
                                                  dtype, dim, 0, 1)
            out[key] = (shape, digest_bytes(raw))
        elif step[0] == "as_dict":
            for name, dim in step[1]:
                raw, shape = by_name[name].get_sharded(name, dim, rank, world)
                out["as_dict:" + name] = (shape, digest_bytes(raw))
    return out


@pytest.mark.parametrize("case", cases.CASES, ids=[c["id"] for c in cases.CASES])
def test_oracle_matches_upstream_outputs(case, golden, case_files):
    paths = case_files(case)
    per_rank = golden["cases"][case["id"]]
    assert len(per_rank) == case["world"]
    for rank, got in enumerate(per_rank):
        want = expected_for_rank(case, paths, rank)
        assert set(got) == set(want)
        for key, rec in got.items():
            if rec is None:
                assert want[key] is None, key
                continue
            shape, _dtype, dig = rec
            assert want[key] is not None, key
            assert list(want[key][0]) == shape, (key, rank)
            assert want[key][1] == dig, (key, rank)


def test_oracle_frame_getitem_matches_upstream(golden):
    for rec in golden["frames"]:
        shape, expr = rec[0], rec[1]
        index = eval(expr, {"slice": slice})
        if len(rec) == 3:
            with pytest.raises((IndexError, ValueError)):
                st_oracle.frame_getitem(shape, index)
        else:
            assert list(st_oracle.frame_getitem(shape, index)) == rec[2:], expr


def test_oracle_header_errors():
    import json
    import struct

    def blob(doc, extra=b""):
        body = json.dumps(doc).encode()
        return struct.pack("<Q", len(body)) + body + extra

    with pytest.raises(st_oracle.HeaderError, match="HeaderTooSmall"):
        st_oracle.parse_header(b"\0" * 7)
    with pytest.raises(st_oracle.HeaderError, match="HeaderTooLarge"):
        st_oracle.parse_header(struct.pack("<Q", 100_000_001) + b"{}")
    with pytest.raises(st_oracle.HeaderError, match="InvalidHeaderLength"):
        st_oracle.parse_header(struct.pack("<Q", 50) + b"{}")
    a = {"dtype": "F16", "shape": [2], "data_offsets": [0, 4]}
    with pytest.raises(st_oracle.HeaderError, match="MetadataIncompleteBuffer"):
        st_oracle.parse_header(blob({"a": a}, b"\0" * 3))
    with pytest.raises(st_oracle.HeaderError, match="InvalidOffset"):
        st_oracle.parse_header(blob({"a": dict(a, data_offsets=[1, 5])}, b"\0" * 8))
    with pytest.raises(st_oracle.HeaderError, match="TensorInvalidInfo"):
        st_oracle.parse_header(blob({"a": dict(a, shape=[3])}, b"\0" * 8))
    hl, tensors, _ = st_oracle.parse_header(blob({"a": a}, b"\0" * 9))  # trailing bytes allowed
    assert list(tensors) == ["a"]
