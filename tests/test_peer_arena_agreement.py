"""Setting up peer arenas is a collective in which any rank may fail (CUDA IPC refused, out of
memory).  Two gloo ranks on CPU with a fake of the native arena calls: whatever fails on one
rank, BOTH ranks get ``PeerArenaUnavailable`` at the same call, everything mapped or allocated
so far is undone, and nobody is left waiting in a collective."""

import json
import os
import sys

import pytest
import torch.distributed as dist
import torch.multiprocessing as mp
from tests.helpers import free_port, rendezvous

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


class FakeArenaLib:
    """Stands in for the fst_arena_* entry points; addresses are made-up integers."""

    def __init__(self, rank, fail):
        self.rank, self.fail = rank, fail
        self.created, self.opened, self.log = set(), set(), []

    def _status(self, call):
        if self.fail == (self.rank, call):
            self.log.append(f"{call}:fail")
            return -5
        return 0

    def fst_arena_create(self, nbytes, out):
        rc = self._status("create")
        if rc == 0:
            out._obj.value = 0x1000_0000 * (self.rank + 1)
            self.created.add(out._obj.value)
        return rc

    def fst_arena_export(self, addr, handle, n):
        handle.raw = int(addr).to_bytes(8, "little") + bytes(n - 8)
        return self._status("export")

    def fst_arena_open_peer(self, handle, n, out):
        rc = self._status("open")
        if rc == 0:
            out._obj.value = int.from_bytes(handle.raw[:8], "little") + 0x1
            self.opened.add(out._obj.value)
        return rc

    def fst_arena_close_peer(self, addr):
        self.opened.discard(int(addr))
        return 0

    def fst_arena_destroy(self, addr):
        self.created.discard(int(addr))
        return 0

    def fst_last_error(self):
        return b"injected by the test"


def _rank(rank, world, port, fail, out_dir):
    sys.path.insert(0, ROOT)
    from fastsafetensors_b200 import _native as nat
    from fastsafetensors_b200 import batch
    from fastsafetensors_b200.st_types import Device

    rdzv = rendezvous(out_dir, port)
    dist.init_process_group("gloo", init_method=rdzv, rank=rank, world_size=world)

    class PG:
        real_pg = dist.group.WORLD

        def rank(self):
            return rank

        def size(self):
            return world

    fake = FakeArenaLib(rank, tuple(fail) if fail else None)
    nat.lib = fake
    dev = Device.from_str(f"cuda:{rank}")
    result = {}
    assert batch.PeerArena.known_unusable(PG(), dev) is False
    try:
        arena = batch.PeerArena.for_group(PG(), 1 << 20, dev)
        result["ok"] = True
        result["peers"] = [hex(p) for p in arena.peer_base]
        arena._alive = False            # destroy() would synchronise a CUDA device
        arena._undo()
    except batch.PeerArenaUnavailable as e:
        result["ok"] = False
        result["error"] = str(e)
        # not tried again for this group, and without any collective
        with pytest.raises(batch.PeerArenaUnavailable):
            batch.PeerArena.for_group(PG(), 1 << 20, dev)
        assert batch.PeerArena.known_unusable(PG(), dev) is True
    result["leaked"] = sorted(fake.created | fake.opened)
    dist.barrier()                       # both ranks are still in step
    with open(os.path.join(out_dir, f"r{rank}.json"), "w") as f:
        json.dump(result, f)
    dist.destroy_process_group()


@pytest.mark.parametrize("fail", [None, (0, "create"), (1, "export"), (1, "open"), (0, "open")],
                         ids=lambda f: "ok" if f is None else f"rank{f[0]}_{f[1]}")
def test_both_ranks_agree(fail, tmp_path):
    port = free_port()
    mp.spawn(_rank, args=(2, port, fail, str(tmp_path)), nprocs=2, join=True)
    got = [json.load(open(tmp_path / f"r{r}.json")) for r in range(2)]
    assert got[0]["leaked"] == [] and got[1]["leaked"] == []
    if fail is None:
        assert got[0]["ok"] and got[1]["ok"]
        assert got[0]["peers"] == ["0x10000000", "0x20000001"]
        assert got[1]["peers"] == ["0x10000001", "0x20000000"]
    else:
        assert not got[0]["ok"] and not got[1]["ok"]
        assert got[0]["error"] == got[1]["error"]
        assert f"rank {fail[0]}" in got[0]["error"]


def test_transport_resolution(monkeypatch):
    from fastsafetensors_b200.file_buffer import resolve_transport
    from fastsafetensors_b200.st_types import Device

    cpu, gpu = Device.from_str("cpu"), Device.from_str("cuda:0")
    monkeypatch.delenv("FST_B200_TRANSPORT", raising=False)
    assert resolve_transport(None, 2, gpu) == "auto"
    assert resolve_transport(None, 8, gpu) == "auto"       # one NVSwitch machine: try peer, fall back
    assert resolve_transport(None, 16, gpu) == "nccl"
    assert resolve_transport("peer", 8, gpu) == "peer"
    assert resolve_transport(None, 2, cpu) == "nccl"
    monkeypatch.setenv("FST_B200_TRANSPORT", "nccl")
    assert resolve_transport(None, 2, gpu) == "nccl"
    with pytest.raises(ValueError):
        resolve_transport("rdma", 2, gpu)
    with pytest.raises(Exception):
        resolve_transport("peer", 2, cpu)
