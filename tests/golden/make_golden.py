"""Generates tests/golden/reference_outputs.json by running UPSTREAM fastsafetensors itself.

Run it where the upstream tree is available (it imports the build made by
``oracle/build_ref.sh`` in ``oracle/_ref``):

    bash oracle/build_ref.sh && python tests/golden/make_golden.py

Inputs are the tiny twins of the benchmark checkpoints, written deterministically by
``tests.synth`` (so the tests can regenerate identical files), plus one crafted
file with mixed dtypes.  Outputs are, per case, the shape, dtype and a 64-bit SHA-256 prefix of
the bytes of every tensor each rank receives from upstream's ``get_tensor`` / ``get_sharded`` /
``get_multi_cols`` / ``push_tensor`` (CPU device, gloo ranks), and upstream's
``TensorFrame.__getitem__`` results for a list of index expressions.
"""

import hashlib
import json
import os
import sys
import tempfile

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, os.path.join(ROOT, "oracle", "_ref"))
sys.path.insert(1, ROOT)

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402
import torch.multiprocessing as mp  # noqa: E402

from tests.golden import cases  # noqa: E402


def digest(t: torch.Tensor) -> str:
    raw = t.detach().contiguous().reshape(-1).view(torch.uint8).numpy().tobytes()
    return hashlib.sha256(raw).hexdigest()[:16]


def record(t) -> list:
    t = t.get_raw() if hasattr(t, "get_raw") else t
    return [list(t.shape), str(t.dtype).replace("torch.", ""), digest(t)]


def run_rank(rank: int, world: int, case: dict, paths: list, port: int, out_dir: str) -> None:
    import fastsafetensors as ref
    from collections import OrderedDict

    pg = None
    if world > 1:
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
        dist.init_process_group("gloo", rank=rank, world_size=world)
        pg = dist.group.WORLD
    loader = ref.SafeTensorsFileLoader(pg if pg is not None else ref.SingleGroup(), "cpu",
                                       nogds=case.get("nogds", True))
    loader.add_filenames(cases.owners(paths, world))
    fb = loader.copy_files_to_device()
    out = {}
    for step in case["steps"]:
        kind = step[0]
        if kind == "plan":       # every tensor by the checkpoint's TP plan
            for name, action in cases.plan(case):
                if action[0] == "shard":
                    out[name] = record(fb.get_sharded(name, action[1]))
                elif action[0] == "replicate":
                    out[name] = record(fb.get_tensor(name))
                else:
                    t = fb.push_tensor(name, action[1] % world)
                    out[name] = record(t) if t is not None else None
        elif kind == "multi_cols":
            _, key, names, dim = step
            out[key] = record(fb.get_multi_cols(names, dim))
        elif kind == "as_dict":
            _, mapping = step
            for name, t in fb.as_dict(OrderedDict(mapping)).items():
                out["as_dict:" + name] = record(t)
    fb.close()
    loader.close()
    with open(os.path.join(out_dir, f"rank{rank}.json"), "w") as f:
        json.dump(out, f)
    if world > 1:
        dist.destroy_process_group()


def frames_golden() -> list:
    from fastsafetensors import TensorFrame
    from fastsafetensors.st_types import DType

    out = []
    for shape, expr in cases.FRAME_INDEXES:
        strides = []
        for i in range(len(shape)):
            s = 1
            for j in range(i + 1, len(shape)):
                s *= shape[j]
            strides.append(s)
        frame = TensorFrame(DType.F16, list(shape), [0, 0], strides, [0] * len(shape), False)
        try:
            got = frame[eval(expr, {"slice": slice})]
            out.append([list(shape), expr, got.shape, got.strides, got.offsets])
        except (IndexError, ValueError) as e:
            out.append([list(shape), expr, type(e).__name__])
    return out


def main() -> None:
    golden = {"frames": frames_golden(), "cases": {}}
    with tempfile.TemporaryDirectory() as tmp:
        for i, case in enumerate(cases.CASES):
            paths = cases.materialize(case, os.path.join(tmp, case["id"]))
            world = case["world"]
            out_dir = os.path.join(tmp, case["id"] + "_out")
            os.makedirs(out_dir)
            if world == 1:
                run_rank(0, 1, case, paths, 0, out_dir)
            else:
                mp.spawn(run_rank, args=(world, case, paths, 29610 + i, out_dir), nprocs=world, join=True)
            golden["cases"][case["id"]] = [
                json.load(open(os.path.join(out_dir, f"rank{r}.json"))) for r in range(world)
            ]
            print(case["id"], "ok", flush=True)
    with open(os.path.join(HERE, "reference_outputs.json"), "w") as f:
        json.dump(golden, f, separators=(",", ":"), sort_keys=True)
        f.write("\n")


if __name__ == "__main__":
    main()
