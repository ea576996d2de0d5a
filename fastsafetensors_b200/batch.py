"""Batched redistribution plan: many tensors, all destination ranks, one gather launch per file
and one exchange per batch.

Upstream moves one tensor per collective (``tensor_factory.py:143,186,258``: a broadcast or a
scatter per tensor, each followed by a device-wide synchronisation).  With file ownership dealt
round-robin the sum of those scatters is a balanced all-to-all: every owner keeps 1/W of what it
read and ships (W-1)/W, every rank receives (W-1)/W of a file-equivalent.  This module lays that
exchange out explicitly:

* ``BatchLayout`` assigns every requested (tensor, destination rank) pair a 256-byte aligned
  slot inside the region ``[owner -> destination]``; every rank computes the same layout from the
  headers alone (all ranks parse all headers);
* the owner fills its ``W`` outgoing regions with ONE gather launch per file
  (``fill_ops``: shards as strided copies, replicated and pushed tensors as flat copies), writing
  its own region straight into the receive buffer;
* one ``all_to_all_single`` with the region sizes as split sizes moves everything; results are
  typed views of the receive buffer.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

from . import shard_plan
from .common import TensorFrame

SLOT_ALIGN = 256

Action = Tuple  # ("shard", dim) | ("replicate",) | ("push", dst_rank)


def _align(n: int) -> int:
    return (n + SLOT_ALIGN - 1) // SLOT_ALIGN * SLOT_ALIGN


@dataclass
class Slot:
    name: str
    offset: int          # inside the [owner -> dst] region
    nbytes: int
    shape: List[int]     # shape of what dst receives (safetensors element counts)


@dataclass
class BatchLayout:
    """Slots of every [owner][dst] region for one batch of requests."""

    world: int
    region_bytes: List[List[int]] = field(default_factory=list)       # [owner][dst]
    slots: List[List[List[Slot]]] = field(default_factory=list)       # [owner][dst] -> slots
    where: Dict[str, Tuple[int, Action]] = field(default_factory=dict)  # name -> (owner, action)

    def __post_init__(self) -> None:
        w = self.world
        self.region_bytes = [[0] * w for _ in range(w)]
        self.slots = [[[] for _ in range(w)] for _ in range(w)]

    def add(self, name: str, frame: TensorFrame, owner: int, action: Action) -> None:
        w = self.world
        bits = frame.dtype.bits
        total = frame.data_offsets[1] - frame.data_offsets[0]
        if action[0] == "shard":
            dim = action[1]
            shard_plan.check_even_split(name, frame.shape[dim], w)
            shape = list(frame.shape)
            shape[dim] = shard_plan.block_size(frame.shape[dim], w)
            rows, row_bytes, _, _ = shard_plan.slice_geometry(frame.shape, bits, dim, 0, shape[dim])
            targets = [(r, rows * row_bytes, shape) for r in range(w)]
        elif action[0] == "replicate":
            targets = [(r, total, list(frame.shape)) for r in range(w)]
        elif action[0] == "push":
            targets = [(action[1], total, list(frame.shape))]
        else:
            raise ValueError(f"unknown action {action!r} for {name}")
        for dst, nbytes, shape in targets:
            off = self.region_bytes[owner][dst]
            self.slots[owner][dst].append(Slot(name, off, nbytes, shape))
            self.region_bytes[owner][dst] = off + _align(nbytes)
        self.where[name] = (owner, action)

    # Buffers as rank `me` sees them.  The region a rank sends to itself never travels: the
    # owner writes it straight into the tail of its receive buffer, behind what the others send.
    def send_sizes(self, me: int) -> List[int]:
        return [0 if d == me else self.region_bytes[me][d] for d in range(self.world)]

    def recv_sizes(self, me: int) -> List[int]:
        return [0 if o == me else self.region_bytes[o][me] for o in range(self.world)]

    def recv_total(self, me: int) -> int:
        return sum(self.recv_sizes(me)) + self.region_bytes[me][me]

    def recv_offset(self, me: int, owner: int) -> int:
        if owner == me:
            return sum(self.recv_sizes(me))
        return sum(self.recv_sizes(me)[:owner])

    def send_offset(self, me: int, dst: int) -> int:
        return sum(self.send_sizes(me)[:dst])

    def fill_ops(self, me: int, frames: Dict[str, TensorFrame], src_addr: Dict[str, int],
                 region_addr: Sequence[int], rotate: bool = False) -> List[shard_plan.Op]:
        """Copies by which owner ``me`` fills its outgoing regions, region by region;
        ``region_addr[dst]`` is where region ``[me -> dst]`` starts (the send buffer, the receive
        buffer for ``dst == me``, or a peer's arena).

        ``rotate`` is for destinations that are peers' memories, where the order of the ops
        matters because the gather kernel works through them in order: regions are then visited
        starting with the owner's own and going round (me+1, me+2, ...), so that at any moment
        different owners are storing to different ranks instead of all of them queueing on one
        rank's NVLink ingress.  (Measured at N = 4: rotated, region by region 4.86 ms per launch;
        tensor by tensor with local and remote stores interleaved 6.14 ms -- warps stalled on
        slow remote stores hold up the local ones.)"""
        ops: List[shard_plan.Op] = []
        w = self.world
        for k in range(w):
            dst = (me + k) % w if rotate else k
            for slot in self.slots[me][dst]:
                if slot.nbytes == 0:
                    continue
                frame = frames[slot.name]
                _, action = self.where[slot.name]
                to = region_addr[dst] + slot.offset
                if action[0] == "shard":
                    lo, hi = shard_plan.shard_bounds(frame.shape[action[1]], w, dst)
                    ops.append(shard_plan.shard_op(src_addr[slot.name], to, frame.shape,
                                                   frame.dtype.bits, action[1], lo, hi))
                else:
                    ops.append((src_addr[slot.name], to, 1, slot.nbytes, 0, 0))
        return ops

    def received(self, me: int) -> List[Tuple[Slot, int]]:
        """(slot, offset in the receive buffer) of everything rank ``me`` ends up with."""
        out: List[Tuple[Slot, int]] = []
        for owner in range(self.world):
            base = self.recv_offset(me, owner)
            for slot in self.slots[owner][me]:
                out.append((slot, base + slot.offset))
        return out


class ShardExchange:
    """One batch of requests, prepared once and runnable many times.

    ``local=False``: this process is rank ``me`` of ``world``; ``run()`` packs what this rank owns
    (gather kernel) and meets the other ranks in one ``all_to_all_single``; ``results()`` are the
    tensors this rank receives.

    ``local=True``: this process owns every file and produces the data of all ``world``
    destinations itself (no transport): ``run()`` is a single gather launch, ``results()`` is a
    list with one ``{name: tensor}`` per destination rank.  This is the owner-side half of the
    exchange run for all destinations at once, e.g. by a single-GPU process that prepares the
    shards of a ``world``-way tensor-parallel group.
    """

    def __init__(self, fb, requests: "Dict[str, Action]", world: int, me: int, local: bool):
        import torch

        from . import _native as nat

        self.fb, self.world, self.me, self.local = fb, world, me, local
        self.names = list(requests)
        self.layout = BatchLayout(world)
        self.frames: Dict[str, TensorFrame] = {}
        src_addr: Dict[str, int] = {}
        self.device = next(l.device for ls in fb.rank_loaders.values() for l in ls)
        for name in self.names:
            rank, lidx = fb._get_rank_lidx(name)
            loader = fb.rank_loaders[rank][lidx]
            self.frames[name] = loader.metadata.tensors[name]
            owner = 0 if local else rank
            self.layout.add(name, self.frames[name], owner, requests[name])
            if owner == me:
                if name not in loader.tensors:
                    raise Exception(f"exchange: tensor {name} was not found, released? lidx={loader.lidx}")
                src_addr[name] = loader.tensors[name].data_ptr()
        torch_dev = "cpu" if self.device.is_cpu else self.device.as_str()
        lay = self.layout
        if local:
            sizes = lay.region_bytes[0]
            self.recv = torch.empty(sum(sizes), dtype=torch.uint8, device=torch_dev)
            self.send = None
            region = [self.recv.data_ptr() + sum(sizes[:d]) for d in range(world)]
        else:
            self.recv = torch.empty(lay.recv_total(me), dtype=torch.uint8, device=torch_dev)
            self.send = torch.empty(sum(lay.send_sizes(me)), dtype=torch.uint8, device=torch_dev)
            region = [self.send.data_ptr() + lay.send_offset(me, d) for d in range(world)]
            region[me] = self.recv.data_ptr() + lay.recv_offset(me, me)
        mine = {n: f for n, f in self.frames.items() if n in src_addr}
        ops = lay.fill_ops(me, mine, src_addr, region) if mine else []
        self.payload_bytes = sum(o[2] * o[3] for o in ops)
        lo, hi = self.recv.data_ptr(), self.recv.data_ptr() + self.recv.numel()
        outgoing = [o for o in ops if not (lo <= o[1] < hi)]
        own = [o for o in ops if lo <= o[1] < hi]
        # (ctypes op array, count, destination base, destination length) per launch.  What has
        # to travel is packed first, so that the exchange can start while this rank's own
        # region is still being packed (see run).
        self.launches = []
        if self.send is not None and outgoing:
            self.launches.append((nat.make_ops(outgoing), len(outgoing), self.send.data_ptr(), self.send.numel()))
        self.n_outgoing_launches = len(self.launches)
        if own:
            self.launches.append((nat.make_ops(own), len(own), self.recv.data_ptr(), self.recv.numel()))

    def _launch_gathers(self, timing: Optional[list], which: Optional[slice] = None) -> None:
        """Enqueue gather launches (all, or ``self.launches[which]``) on torch's current stream.
        With ``timing`` a list, a pair of CUDA events brackets every launch and is appended."""
        from . import _native as nat

        todo = self.launches if which is None else self.launches[which]
        if self.device.is_cpu:
            for arr, n, _, _ in todo:
                nat.check(nat.lib.fst_gather_host(arr, n, 8), "fst_gather_host")
            return
        stream = self.fb.framework.current_stream(self.device)
        for arr, n, base, length in todo:
            if timing is not None:
                import torch

                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record()
            nat.check(nat.lib.fst_gather(arr, n, 0, 0, base, length, stream), "fst_gather")
            if timing is not None:
                b.record()
                timing.append((a, b))

    def run(self, timing: Optional[list] = None) -> None:
        """Pack and exchange.  The outgoing regions are packed first and the ``all_to_all`` is
        started asynchronously; this rank's own region is packed while the exchange runs (the two
        write disjoint parts of the receive buffer); then the stream waits for the exchange."""
        if self.local:
            self._launch_gathers(timing)
            return
        import torch.distributed as dist

        k = self.n_outgoing_launches
        self._launch_gathers(timing, slice(0, k))
        lay, me = self.layout, self.me
        incoming = sum(lay.recv_sizes(me))
        work = dist.all_to_all_single(self.recv[:incoming], self.send, lay.recv_sizes(me),
                                      lay.send_sizes(me), group=self.fb.pg.real_pg, async_op=True)
        self._launch_gathers(timing, slice(k, None))
        work.wait()

    def _view(self, slot: Slot, off: int):
        from .frameworks._torch import TorchTensor, dtype_convert

        frame = self.frames[slot.name]
        native = self.fb.framework.get_native_shape(frame.dtype, slot.shape)
        t = self.recv[off: off + slot.nbytes].view(dtype_convert[frame.dtype]).reshape(native)
        return TorchTensor(self.device, frame.dtype, t)

    def results(self):
        lay = self.layout
        if not self.local:
            return {slot.name: self._view(slot, off) for slot, off in lay.received(self.me)}
        out = []
        sizes = lay.region_bytes[0]
        for dst in range(self.world):
            base = sum(sizes[:dst])
            out.append({s.name: self._view(s, base + s.offset) for s in lay.slots[0][dst]})
        return out


class PeerArenaUnavailable(RuntimeError):
    """The ranks of a group cannot map each other's memory (different machines, CUDA IPC refused,
    out of memory on one rank).  Every rank of the group raises it at the same call."""


class PeerArena:
    """This rank's receive arena (plain ``cudaMalloc``, exported over CUDA IPC) and the mappings
    of every peer's arena.  Creating one is a collective (the handles are all-gathered), and
    mapping a peer's arena costs tens of milliseconds per peer, so arenas are kept per process
    group (``PeerArena.for_group``) and reused by later exchanges; what a rank receives is copied
    out of the arena into its own tensor memory.

    A failure on one rank must not leave the others waiting in a collective, so the constructor
    never raises between its collectives: each rank carries its own error through the two
    all-gathers (handles, then the outcome of mapping them), all ranks undo what they did, and all
    raise ``PeerArenaUnavailable`` together."""

    _cache: Dict[Tuple[int, str], "PeerArena"] = {}
    _failed: Dict[Tuple[int, str], str] = {}

    def __init__(self, pg, nbytes: int, device):
        import ctypes
        import socket

        import torch.distributed as dist

        from . import _native as nat

        self._nat = nat
        self.pg = pg
        self.nbytes = max(int(nbytes), 256)
        self.device = device
        self.rank, self.world = pg.rank(), pg.size()
        self.address = 0
        self.peer_base: List[int] = []
        self._alive = False
        err: Optional[str] = None
        handle = ctypes.create_string_buffer(nat.ARENA_HANDLE_BYTES)
        try:
            addr = ctypes.c_uint64(0)
            nat.check(nat.lib.fst_arena_create(self.nbytes, ctypes.byref(addr)), "fst_arena_create")
            self.address = addr.value
            nat.check(nat.lib.fst_arena_export(self.address, handle, nat.ARENA_HANDLE_BYTES), "fst_arena_export")
        except nat.NativeError as e:
            err = str(e)
        said: List[Optional[tuple]] = [None] * self.world
        dist.all_gather_object(said, (err, handle.raw, socket.gethostname()), group=pg.real_pg)
        problems = [f"rank {r}: {m[0]}" for r, m in enumerate(said) if m[0]]
        if not problems and len({m[2] for m in said}) > 1:
            problems = ["ranks are on different machines: " + ", ".join(sorted({m[2] for m in said}))]
        if not problems:
            mapped: List[int] = []
            try:
                for r, m in enumerate(said):
                    if r == self.rank:
                        mapped.append(self.address)
                        continue
                    p = ctypes.c_uint64(0)
                    buf = ctypes.create_string_buffer(m[1], nat.ARENA_HANDLE_BYTES)
                    nat.check(nat.lib.fst_arena_open_peer(buf, nat.ARENA_HANDLE_BYTES, ctypes.byref(p)),
                              "fst_arena_open_peer")
                    mapped.append(p.value)
            except nat.NativeError as e:
                err = str(e)
            self.peer_base = mapped          # what was mapped so far, for the undo below
            outcome: List[Optional[str]] = [None] * self.world
            dist.all_gather_object(outcome, err, group=pg.real_pg)
            problems = [f"rank {r}: {m}" for r, m in enumerate(outcome) if m]
        if problems:
            self._undo()
            raise PeerArenaUnavailable("peer arenas cannot be set up: " + "; ".join(problems))
        self._alive = True

    def _undo(self) -> None:
        """Unmap what this rank mapped, wait until every rank has, free this rank's arena."""
        import torch.distributed as dist

        for r, p in enumerate(self.peer_base):
            if r != self.rank and p:
                self._nat.lib.fst_arena_close_peer(p)
        self.peer_base = []
        dist.barrier(group=self.pg.real_pg)
        if self.address:
            self._nat.lib.fst_arena_destroy(self.address)
            self.address = 0

    @classmethod
    def for_group(cls, pg, nbytes: int, device) -> "PeerArena":
        """The group's arena, grown if needed.  ``nbytes`` must be the same on every rank (callers
        pass the largest need of any rank), so that all ranks decide alike whether to grow.
        A group whose arenas could not be set up once is not tried again."""
        key = (id(pg.real_pg), device.as_str())
        if key in cls._failed:
            raise PeerArenaUnavailable(cls._failed[key])
        cur = cls._cache.get(key)
        if cur is not None and cur.nbytes >= nbytes:
            return cur
        if cur is not None:
            cur.destroy()
            del cls._cache[key]
        grown = max(int(nbytes * 1.25), 64 << 20)
        try:
            cls._cache[key] = cls(pg, (grown + (1 << 21) - 1) >> 21 << 21, device)
        except PeerArenaUnavailable as e:
            cls._failed[key] = str(e)
            raise
        return cls._cache[key]

    @classmethod
    def known_unusable(cls, pg, device) -> bool:
        """True once setting up arenas for this group has failed (on every rank alike)."""
        return (id(pg.real_pg), device.as_str()) in cls._failed

    @classmethod
    def release_all(cls) -> None:
        """Destroy every cached arena.  Collective per process group (each ends in a barrier)."""
        for arena in list(cls._cache.values()):
            arena.destroy()
        cls._cache.clear()

    def destroy(self) -> None:
        """Unmap the peers, wait for every rank to have done so, then free this rank's arena."""
        import torch

        if not self._alive:
            return
        self._alive = False
        torch.cuda.synchronize()
        self._undo()

    def view(self, nbytes: int):
        """Non-owning ``torch.uint8`` view of the first ``nbytes`` of this rank's arena."""
        import torch

        class _Span:
            __cuda_array_interface__ = {
                "shape": (max(int(nbytes), 1),), "typestr": "|u1", "data": (self.address, False), "version": 2,
            }

        return torch.as_tensor(_Span(), device=self.device.as_str())[: int(nbytes)]


class PeerShardExchange(ShardExchange):
    """``ShardExchange`` whose transport is the gather kernel itself.

    Every rank has a peer arena (see ``PeerArena``) that the other ranks have mapped.  The
    owner's single gather launch stores each shard directly where it is needed: its own region
    into its receive buffer, every other region into the arena of the destination rank, over
    NVLink, with ordinary 16-byte stores.  No send buffer and no ``all_to_all``.  One step is

        barrier (all ranks have emptied their arenas) -> gather launch -> barrier (all ranks'
        kernels are complete) -> copy of what arrived from the arena into this rank's own buffer

    where a barrier is an 8-byte all-reduce on the same stream, so nothing synchronises the host.
    """

    def __init__(self, fb, requests: "Dict[str, Action]", world: int, me: int):
        import torch

        from . import _native as nat

        self.fb, self.world, self.me, self.local = fb, world, me, False
        self.names = list(requests)
        self.layout = BatchLayout(world)
        self.frames = {}
        src_addr: Dict[str, int] = {}
        self.device = next(l.device for ls in fb.rank_loaders.values() for l in ls)
        if self.device.is_cpu:
            raise Exception("the peer transport needs CUDA devices")
        for name in self.names:
            rank, lidx = fb._get_rank_lidx(name)
            loader = fb.rank_loaders[rank][lidx]
            self.frames[name] = loader.metadata.tensors[name]
            self.layout.add(name, self.frames[name], rank, requests[name])
            if rank == me:
                if name not in loader.tensors:
                    raise Exception(f"exchange: tensor {name} was not found, released? lidx={loader.lidx}")
                src_addr[name] = loader.tensors[name].data_ptr()
        lay = self.layout
        # the arena holds what the OTHER ranks send; every rank sizes it for the neediest rank
        need = max(sum(lay.recv_sizes(r)) for r in range(world))
        self.arena = PeerArena.for_group(fb.pg, need, self.device)
        self.incoming = sum(lay.recv_sizes(me))
        self.recv = torch.empty(lay.recv_total(me), dtype=torch.uint8, device=self.device.as_str())
        self.send = None
        self._arena_view = self.arena.view(self.incoming)
        # region [me -> d]: d's arena at the offset where d expects owner `me`; own region: recv
        region = [self.arena.peer_base[d] + lay.recv_offset(d, me) for d in range(world)]
        region[me] = self.recv.data_ptr() + lay.recv_offset(me, me)
        mine = {n: f for n, f in self.frames.items() if n in src_addr}
        ops = lay.fill_ops(me, mine, src_addr, region, rotate=True) if mine else []
        self.payload_bytes = sum(o[2] * o[3] for o in ops)
        self.launches = [(nat.make_ops(ops), len(ops), 0, 0)] if ops else []
        self._flag = torch.zeros(1, dtype=torch.int32, device=self.device.as_str())

    def run(self, timing: Optional[list] = None) -> None:
        import torch.distributed as dist

        group = self.fb.pg.real_pg
        dist.all_reduce(self._flag, group=group)      # every rank has emptied its arena
        self._launch_gathers(timing)
        dist.all_reduce(self._flag, group=group)      # every rank's kernel is complete
        if self.incoming:
            self.recv[: self.incoming].copy_(self._arena_view)

    def finish(self) -> None:
        """Kept for callers of the earlier interface; the arena now outlives the exchange."""
