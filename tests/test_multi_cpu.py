"""Multi-rank path on CPU: gloo ranks, device "cpu", checked against upstream's recorded
per-rank outputs (shards, broadcasts, column groups, pushes) for the same requests."""

import json
import os
import sys
from collections import OrderedDict

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from tests.golden import cases

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _rank_main(rank, world, case, paths, port, out_dir, batched=False, backend="gloo", transport="nccl"):
    sys.path.insert(0, ROOT)
    import fastsafetensors_b200 as fst
    from fastsafetensors_b200 import cpp
    from tests.helpers import record

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    if backend == "nccl":
        torch.cuda.set_device(rank)
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device(f"cuda:{rank}"))
        device = f"cuda:{rank}"
    else:
        dist.init_process_group("gloo", rank=rank, world_size=world)
        device = "cpu"
    loader = fst.SafeTensorsFileLoader(dist.group.WORLD, device, nogds=True, max_threads=2, slot_kb=64)
    loader.add_filenames(cases.owners(paths, world))
    fb = loader.copy_files_to_device()
    out = {}
    for step in case["steps"]:
        if step[0] == "plan" and batched:
            # the whole plan in one batched exchange (tiny batches force several rounds)
            plan = OrderedDict((n, (a[0], a[1] % world) if a[0] == "push" else a) for n, a in cases.plan(case))
            got = fb.exchange(plan, max_batch_bytes=1 << 20, transport=transport)
            for name, action in plan.items():
                if action[0] == "push" and action[1] != rank:
                    assert name not in got
                    out[name] = None
                else:
                    out[name] = record(got[name])
        elif step[0] == "plan":
            for name, action in cases.plan(case):
                if action[0] == "shard":
                    out[name] = record(fb.get_sharded(name, action[1]))
                elif action[0] == "replicate":
                    out[name] = record(fb.get_tensor(name))
                else:
                    t = fb.push_tensor(name, action[1] % world)
                    out[name] = record(t) if t is not None else None
        elif step[0] == "multi_cols":
            out[step[1]] = record(fb.get_multi_cols(step[2], step[3]))
        elif step[0] == "as_dict":
            for name, t in fb.as_dict(OrderedDict(step[1])).items():
                out["as_dict:" + name] = record(t)
    # every file was requested in full by the "plan" step: its image must be gone already
    if list(case["steps"]) == [("plan",)] and not case.get("skip"):
        assert all(f.gbuf is None for fs in fb.rank_loaders.values() for f in fs)
    fb.close()
    loader.close()
    assert loader.framework.get_mem_used() == 0
    assert cpp.get_cpp_metrics().bounce_buffer_bytes == 0
    with open(os.path.join(out_dir, f"rank{rank}.json"), "w") as f:
        json.dump(out, f)
    dist.destroy_process_group()


MULTI = [c for c in cases.CASES if c["world"] > 1 and c["id"] in
         ("llama3_8b_w2_cols", "llama2_13b_w4", "mixtral_w8", "crafted_w2")]


@pytest.mark.parametrize("batched", [False, True], ids=["per_tensor", "batched"])
@pytest.mark.parametrize("case", MULTI, ids=[c["id"] for c in MULTI])
def test_gloo_ranks_match_upstream(case, batched, golden, case_files, tmp_path):
    if batched and case["steps"][0][0] != "plan":
        pytest.skip("as_dict in the per-tensor run already goes through the batched exchange")
    paths = case_files(case)
    world = case["world"]
    port = 29700 + 2 * cases.CASES.index(case) + int(batched)
    mp.spawn(_rank_main, args=(world, case, paths, port, str(tmp_path), batched), nprocs=world, join=True)
    for rank in range(world):
        got = json.load(open(tmp_path / f"rank{rank}.json"))
        assert got == golden["cases"][case["id"]][rank], f"rank {rank}"
