"""Batched redistribution plan: many tensors, all destination ranks, one gather launch per file
and chunk, transfers overlapped with the reads of the files still to come.

Upstream moves one tensor per collective (``tensor_factory.py:143,186,258``: a broadcast or a
scatter per tensor, each followed by a device-wide synchronisation).  With file ownership dealt
round-robin the sum of those scatters is a balanced all-to-all: every owner keeps 1/W of what it
read and ships (W-1)/W, every rank receives (W-1)/W of a file-equivalent.  This module lays that
exchange out explicitly:

* ``BatchLayout`` assigns every requested (tensor, destination rank) pair a 256-byte aligned
  slot inside the region ``[owner -> destination]``; every rank computes the same layout from the
  headers alone (all ranks parse all headers);
* the owner fills its ``W`` outgoing regions with one gather launch per chunk
  (``fill_ops``: shards as strided copies, replicated and pushed tensors as flat copies), writing
  its own region straight into the receive buffer;
* ``ShardExchange``: one ``all_to_all_single`` per chunk (by default a chunk is a round: the
  j-th file of every owner) with the region sizes as split sizes moves the data while the next
  round is being packed (and, with deferred reads, read);
* ``PeerShardExchange``: no collective moves data at all -- the gather launches store into the
  destination ranks' memory over NVLink, and one small all-reduce closes the exchange;
* results are typed views of one receive buffer.
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
                 region_addr: Sequence[int], rotate=False) -> List[shard_plan.Op]:
        """Copies by which owner ``me`` fills its outgoing regions, region by region;
        ``region_addr[dst]`` is where region ``[me -> dst]`` starts (the send buffer, the receive
        buffer for ``dst == me``, or a peer's arena).

        ``rotate`` is for destinations that are peers' memories, where the order of the ops
        matters because the gather kernel works through them in order.  ``True``: regions are
        visited starting with the owner's own and going round (me+1, me+2, ...), so that at any
        moment different owners are storing to different ranks instead of all of them queueing
        on one rank's NVLink ingress.  ``"interleave"``: the own region first, then the peers'
        regions tensor by tensor (measured at four ranks, peer stores in a launch of their own:
        12.9 ms per step against 13.2 ms region by region)."""
        ops: List[shard_plan.Op] = []
        w = self.world

        def op_for(slot: Slot, dst: int) -> shard_plan.Op:
            frame = frames[slot.name]
            _, action = self.where[slot.name]
            to = region_addr[dst] + slot.offset
            if action[0] == "shard":
                lo, hi = shard_plan.shard_bounds(frame.shape[action[1]], w, dst)
                return shard_plan.shard_op(src_addr[slot.name], to, frame.shape, frame.dtype.bits, action[1], lo, hi)
            return (src_addr[slot.name], to, 1, slot.nbytes, 0, 0)

        if rotate == "interleave":
            # the owner's own region first, then tensor by tensor: the slots of one tensor in all
            # the other destinations, starting with the next rank.  Every owner then stores to all
            # its peers at once, so each rank's NVLink ingress is shared evenly whatever the
            # owners' relative progress.
            for slot in self.slots[me][me]:
                if slot.nbytes:
                    ops.append(op_for(slot, me))
            by_name: List[Dict[str, Slot]] = [{s.name: s for s in self.slots[me][d]} for d in range(w)]
            order: List[str] = []
            seen = set()
            for d in range(w):
                for s in self.slots[me][d]:
                    if s.name not in seen:
                        seen.add(s.name)
                        order.append(s.name)
            for name in order:
                for k in range(1, w):
                    dst = (me + k) % w
                    slot = by_name[dst].get(name)
                    if slot is not None and slot.nbytes:
                        ops.append(op_for(slot, dst))
            return ops
        for k in range(w):
            dst = (me + k) % w if rotate else k
            for slot in self.slots[me][dst]:
                if slot.nbytes == 0:
                    continue
                ops.append(op_for(slot, dst))
        return ops

    def received(self, me: int) -> List[Tuple[Slot, int]]:
        """(slot, offset in the receive buffer) of everything rank ``me`` ends up with."""
        out: List[Tuple[Slot, int]] = []
        for owner in range(self.world):
            base = self.recv_offset(me, owner)
            for slot in self.slots[owner][me]:
                out.append((slot, base + slot.offset))
        return out


def cut_into_chunks(fb, requests: "Dict[str, Action]", world: int, chunk_bytes: int) -> List[List[str]]:
    """Order of work for one exchange: requests grouped by *round* (round j = the j-th file of
    every owner rank, i.e. the files the ranks read at the same time), each round cut, in request
    order, into chunks in which no owner sends more than ``chunk_bytes``.  Every rank computes the
    same chunks from the headers alone."""
    by_round: Dict[int, List[str]] = {}
    for name in requests:
        _, lidx = fb._get_rank_lidx(name)
        by_round.setdefault(lidx, []).append(name)
    chunks: List[List[str]] = []
    for lidx in sorted(by_round):
        volume: Dict[int, int] = {}
        cur: List[str] = []
        for name in by_round[lidx]:
            rank, _ = fb._get_rank_lidx(name)
            frame = fb.rank_loaders[rank][lidx].metadata.tensors[name]
            nbytes = frame.data_offsets[1] - frame.data_offsets[0]
            cost = nbytes * (world if requests[name][0] == "replicate" else 1)
            if cur and volume.get(rank, 0) + cost > chunk_bytes:
                chunks.append(cur)
                cur, volume = [], {}
            cur.append(name)
            volume[rank] = volume.get(rank, 0) + cost
        if cur:
            chunks.append(cur)
    return chunks


@dataclass
class _Chunk:
    names: List[str]
    layout: BatchLayout
    recv_base: int                 # offset of this chunk's part of the receive buffer
    recv_bytes: int
    send_bytes: int
    launches: Optional[list] = None    # [(op array, count, dst base, dst length, outgoing?)]
    payload: int = 0


class ShardExchange:
    """The requests of one ``exchange`` / ``shard_locally`` call, prepared once, runnable many
    times.

    The requests are cut into chunks (``cut_into_chunks``).  ``run()`` takes the chunks in order:
    wait until this rank's file of the chunk has been read (a no-op unless the loader was asked
    not to wait), pack what this rank owns with the gather kernel, start the chunk's
    ``all_to_all_single`` asynchronously, go on to the next chunk.  So the gather of chunk k+1
    runs while NVLink still carries chunk k, and with ``copy_files_to_device(wait=False)`` both
    run while the reader is still filling the files of later rounds.  All chunks receive into
    ONE buffer (allocated up front from the headers), sends go through a ring of two chunk-sized
    buffers.

    ``local=False``: this process is rank ``me`` of ``world``; ``results()`` are the tensors this
    rank receives.  ``local=True``: this process owns every file and produces the data of all
    ``world`` destinations itself (no transport, one gather launch per file); ``results()`` is a
    list with one ``{name: tensor}`` per destination rank -- the owner-side half of the exchange
    run for all destinations at once, e.g. by a single-GPU process that prepares the shards of a
    ``world``-way tensor-parallel group.
    """

    SEND_SLOTS = 2

    def __init__(self, fb, requests: "Dict[str, Action]", world: int, me: int, local: bool,
                 chunk_bytes: Optional[int] = None):
        import torch

        self.fb, self.world, self.me, self.local = fb, world, me, local
        self.requests = dict(requests)
        self.names = list(requests)
        self.frames: Dict[str, TensorFrame] = {}
        self.device = next(l.device for ls in fb.rank_loaders.values() for l in ls)
        if chunk_bytes is None:
            chunk_bytes = (1 << 62) if local else default_chunk_bytes()
        self.chunks: List[_Chunk] = []
        recv_total, send_max = 0, 0
        for names in cut_into_chunks(fb, requests, world, chunk_bytes):
            lay = BatchLayout(world)
            for name in names:
                rank, lidx = fb._get_rank_lidx(name)
                frame = fb.rank_loaders[rank][lidx].metadata.tensors[name]
                self.frames[name] = frame
                lay.add(name, frame, 0 if local else rank, requests[name])
            recv = sum(lay.region_bytes[0]) if local else lay.recv_total(me)
            send = 0 if local else sum(lay.send_sizes(me))
            self.chunks.append(_Chunk(names, lay, recv_total, recv, send))
            recv_total += recv
            send_max = max(send_max, send)
        torch_dev = "cpu" if self.device.is_cpu else self.device.as_str()
        self.recv = torch.empty(recv_total, dtype=torch.uint8, device=torch_dev)
        self.send_slot_bytes = send_max
        self.send = None if local else torch.empty(self.SEND_SLOTS * send_max, dtype=torch.uint8,
                                                    device=torch_dev)
        self._slot_work: List[Optional[object]] = [None] * self.SEND_SLOTS
        self.payload_bytes = 0          # bytes this rank's gather launches move (known after run)
        # bytes this rank sends to other ranks over the whole exchange
        self.egress_bytes = 0 if local else sum(
            ch.layout.region_bytes[me][d] for ch in self.chunks for d in range(world) if d != me)

    # ------------------------------------------------------------------ preparation of one chunk
    def _prepare(self, index: int) -> _Chunk:
        """Op tables of chunk ``index`` (built once).  Touches the tensors of the files this rank
        owns in the chunk, which completes their reads if those were deferred."""
        ch = self.chunks[index]
        if ch.launches is not None:
            return ch
        from . import _native as nat

        fb, lay, me = self.fb, ch.layout, self.me
        src_addr: Dict[str, int] = {}
        for name in ch.names:
            rank, lidx = fb._get_rank_lidx(name)
            if self.local or rank == me:
                loader = fb.rank_loaders[rank][lidx]
                tensors = loader.tensors
                if name not in tensors:
                    raise Exception(f"exchange: tensor {name} was not found, released? lidx={loader.lidx}")
                src_addr[name] = tensors[name].data_ptr()
        recv_ptr = self.recv.data_ptr() + ch.recv_base
        slot = index % self.SEND_SLOTS
        if self.local:
            sizes = lay.region_bytes[0]
            region = [recv_ptr + sum(sizes[:d]) for d in range(self.world)]
        else:
            send_ptr = self.send.data_ptr() + slot * self.send_slot_bytes
            region = [send_ptr + lay.send_offset(me, d) for d in range(self.world)]
            region[me] = recv_ptr + lay.recv_offset(me, me)
        mine = {n: self.frames[n] for n in src_addr}
        ops = lay.fill_ops(me, mine, src_addr, region) if mine else []
        ch.payload = sum(o[2] * o[3] for o in ops)
        lo, hi = recv_ptr, recv_ptr + ch.recv_bytes
        outgoing = [o for o in ops if not (lo <= o[1] < hi)]
        own = [o for o in ops if lo <= o[1] < hi]
        ch.launches = []
        if outgoing:       # what has to travel is packed first, so that the exchange can start
            ch.launches.append((nat.pack_ops(outgoing), len(outgoing), send_ptr, ch.send_bytes, True))
        if own:
            ch.launches.append((nat.pack_ops(own), len(own), recv_ptr, ch.recv_bytes, False))
        return ch

    def _launch(self, ch: _Chunk, outgoing: bool, timing: Optional[list]) -> None:
        """Enqueue the chunk's gather launches of one kind on torch's current stream.  With
        ``timing`` a list, a pair of CUDA events brackets every launch and is appended."""
        from . import _native as nat

        for packed, n, base, length, is_out in ch.launches:
            if is_out != outgoing:
                continue
            if self.device.is_cpu:
                nat.check(nat.lib.fst_gather_host(packed.pointer, n, 8), "fst_gather_host")
                continue
            stream = self.fb.framework.current_stream(self.device)
            if timing is not None:
                import torch

                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record()
            nat.check(nat.lib.fst_gather(packed.pointer, n, 0, 0, base, length, stream), "fst_gather")
            if timing is not None:
                b.record()
                timing.append((a, b))

    # ------------------------------------------------------------------ the exchange
    def run(self, timing: Optional[list] = None, after_chunk=None) -> None:
        """Pack and exchange chunk by chunk.  ``after_chunk(names)`` is called when a chunk's
        work has been queued (the caller releases file images there)."""
        payload = 0
        for index in range(len(self.chunks)):
            ch = self._prepare(index)
            payload += ch.payload
            if self.local:
                self._launch(ch, False, timing)
            else:
                self._run_chunk(index, ch, timing)
            if after_chunk is not None:
                after_chunk(ch.names)
        self.payload_bytes = payload
        for slot, work in enumerate(self._slot_work):
            if work is not None:
                work.wait()
                self._slot_work[slot] = None

    def _run_chunk(self, index: int, ch: _Chunk, timing: Optional[list]) -> None:
        import torch.distributed as dist

        lay, me = ch.layout, self.me
        slot = index % self.SEND_SLOTS
        if self._slot_work[slot] is not None:
            # the collective that last read this send slot must be done before the gather
            # overwrites it (a stream-side wait for NCCL)
            self._slot_work[slot].wait()
            self._slot_work[slot] = None
        self._launch(ch, True, timing)
        incoming = sum(lay.recv_sizes(me))
        recv = self.recv[ch.recv_base: ch.recv_base + incoming]
        send = self.send[slot * self.send_slot_bytes: slot * self.send_slot_bytes + ch.send_bytes]
        self._slot_work[slot] = dist.all_to_all_single(
            recv, send, lay.recv_sizes(me), lay.send_sizes(me), group=self.fb.pg.real_pg, async_op=True)
        # this rank's own region is packed while the exchange runs (disjoint part of the buffer)
        self._launch(ch, False, timing)

    # ------------------------------------------------------------------ results
    def _view(self, slot: Slot, off: int):
        from .frameworks._torch import TorchTensor, dtype_convert

        frame = self.frames[slot.name]
        native = self.fb.framework.get_native_shape(frame.dtype, slot.shape)
        t = self.recv[off: off + slot.nbytes].view(dtype_convert[frame.dtype]).reshape(native)
        return TorchTensor(self.device, frame.dtype, t)

    def results(self):
        if not self.local:
            out = {}
            for ch in self.chunks:
                for slot, off in ch.layout.received(self.me):
                    out[slot.name] = self._view(slot, ch.recv_base + off)
            return out
        per_dst: List[Dict[str, object]] = [{} for _ in range(self.world)]
        for ch in self.chunks:
            sizes = ch.layout.region_bytes[0]
            for dst in range(self.world):
                base = ch.recv_base + sum(sizes[:dst])
                for s in ch.layout.slots[0][dst]:
                    per_dst[dst][s.name] = self._view(s, base + s.offset)
        return per_dst


def peer_remote_ctas(world: int, device_index: int = 0) -> int:
    """Grid bound of the launch that stores into the peers' arenas while this rank's own region
    is packed by a second launch beside it; 0 = one launch does both, region after region.
    ``FST_B200_PEER_REMOTE_CTAS`` sets it.  The default is ``world // 2`` CTAs per SM (at most
    four, the kernel's residency): enough stores in flight to fill NVLink towards ``world - 1``
    peers, and CTA slots left to the own region.  Measured on B200, ms per step of a 38 GB
    checkpoint -- two ranks: 16.6 with one launch, 14.9 / 13.9 / 15.7 / 15.4 with 74 / 148 / 296 /
    592 CTAs; four ranks: 14.0 with one launch, 14.2 / 12.9 / 13.0 / 13.6 with 148 / 296 / 444 /
    592 CTAs."""
    import os

    env = os.environ.get("FST_B200_PEER_REMOTE_CTAS")
    if env is not None:
        return max(0, int(env))
    import torch

    sms = int(torch.cuda.get_device_properties(device_index).multi_processor_count)
    return sms * max(1, min(4, world // 2))


def default_chunk_bytes() -> int:
    """Outgoing bytes per owner and chunk of an exchange over NCCL.  Default: no cut below a
    round (one file per owner).  ``FST_B200_EXCHANGE_CHUNK_MB`` cuts rounds further; on B200 that
    measured slower, not faster (1 GiB chunks: 31 ms against 16 ms per step at two ranks, 48 ms at
    four): the gather launches of the next chunk fill every SM and NCCL's copy kernels, which
    need a few of them, queue behind."""
    import os

    env = os.environ.get("FST_B200_EXCHANGE_CHUNK_MB")
    return (max(1, int(env)) << 20) if env else (1 << 62)


class PeerArenaUnavailable(RuntimeError):
    """The ranks of a group cannot map each other's memory (different machines, CUDA IPC refused,
    out of memory on one rank).  Every rank of the group raises it at the same call."""


class PeerArena:
    """This rank's receive arena for one exchange (plain ``cudaMalloc``, exported over CUDA IPC)
    and the mappings of every peer's arena.  What a rank receives stays in its arena: the result
    tensors are views of it and keep it alive, so nothing is copied out.

    Creating one is a collective (the handles are all-gathered).  A failure on one rank must not
    leave the others waiting in a collective, so the constructor never raises between its
    collectives: each rank carries its own error through the two all-gathers (handles, then the
    outcome of mapping them), all ranks undo what they did, and all raise
    ``PeerArenaUnavailable`` together.  ``close_peers`` (collective) unmaps the peers once the
    exchange is over; from then on every arena belongs to its own rank alone and is freed when
    the last tensor over it is gone."""

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
        self._shared = False          # peers may still have this rank's arena mapped
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
        self._shared = True

    def _unmap_peers(self) -> None:
        for r, p in enumerate(self.peer_base):
            if r != self.rank and p:
                self._nat.lib.fst_arena_close_peer(p)
        self.peer_base = []

    def _undo(self) -> None:
        """Unmap what this rank mapped, wait until every rank has, free this rank's arena."""
        import torch.distributed as dist

        self._unmap_peers()
        dist.barrier(group=self.pg.real_pg)
        self._shared = False
        self._free()

    def _free(self) -> None:
        if self.address:
            self._nat.lib.fst_arena_destroy(self.address)
            self.address = 0

    @classmethod
    def for_group(cls, pg, nbytes: int, device) -> "PeerArena":
        """A new arena of ``nbytes`` on every rank of the group (collective; ``nbytes`` must be
        the same on every rank).  A group whose arenas could not be set up once is not tried
        again: the failure is remembered and raised at once, without a collective."""
        key = (id(pg.real_pg), device.as_str())
        if key in cls._failed:
            raise PeerArenaUnavailable(cls._failed[key])
        try:
            return cls(pg, (int(nbytes) + (1 << 21) - 1) >> 21 << 21, device)
        except PeerArenaUnavailable as e:
            cls._failed[key] = str(e)
            raise

    @classmethod
    def known_unusable(cls, pg, device) -> bool:
        """True once setting up arenas for this group has failed (on every rank alike)."""
        return (id(pg.real_pg), device.as_str()) in cls._failed

    def close_peers(self) -> None:
        """Collective: the work queued so far is drained, every rank unmaps its peers, and all
        meet in a barrier.  After it nobody but the owner can touch an arena."""
        import torch
        import torch.distributed as dist

        if not self._alive or not self._shared:
            return
        torch.cuda.synchronize()
        self._unmap_peers()
        dist.barrier(group=self.pg.real_pg)
        self._shared = False

    def destroy(self) -> None:
        """Collective unless ``close_peers`` has run: unmap, meet, free this rank's arena."""
        if not self._alive:
            return
        self.close_peers()
        self._alive = False
        self._free()

    def __del__(self) -> None:
        # the last tensor over the arena is gone.  If the peers were never told to unmap it
        # (an exchange abandoned half-way), the memory is left to the process's teardown.
        try:
            if self._alive and not self._shared:
                self._alive = False
                self._free()
        except Exception:  # noqa: BLE001
            pass

    def view(self, nbytes: int):
        """``torch.uint8`` tensor over the first ``nbytes`` of this rank's arena.  The tensor
        (and every view derived from it) keeps the arena object alive."""
        import torch

        return torch.as_tensor(_ArenaSpan(self, nbytes), device=self.device.as_str())[: int(nbytes)]


class _ArenaSpan:
    """What ``torch.as_tensor`` wraps: the arena's bytes through the CUDA array interface.  torch
    keeps this object for as long as the storage lives, and the object keeps the arena."""

    def __init__(self, arena: "PeerArena", nbytes: int):
        self.owner = arena
        self.__cuda_array_interface__ = {
            "shape": (max(int(nbytes), 1),), "typestr": "|u1", "data": (arena.address, False), "version": 2,
        }


class PeerShardExchange:
    """The exchange with the gather kernel itself as transport.

    Every rank has a peer arena (see ``PeerArena``) sized for everything it will receive, which
    the other ranks have mapped.  The requests are cut into chunks round by round, as in
    ``ShardExchange``; per chunk the owner's ONE gather launch stores each shard directly where
    it is needed: its own region into its own arena, every other region into the arena of the
    destination rank, over NVLink, with ordinary 16-byte stores.  No send buffer, no
    ``all_to_all``, no copy out of the arena: the results are views of it.  After the last
    chunk one 4-byte all-reduce on the same stream tells every rank that all kernels (and with
    them all peer stores) are complete; nothing synchronises the host.  With deferred reads
    (``copy_files_to_device(wait=False)``) the launches of round k run while the reader fills the
    files of round k+1.

    Regions are disjoint per (owner, destination) pair, so ``run()`` may be repeated.
    """

    def __init__(self, fb, requests: "Dict[str, Action]", world: int, me: int,
                 chunk_bytes: Optional[int] = None, arena=None):
        """``arena``: an object with ``address``, ``nbytes``, ``peer_base`` and ``view`` to use
        instead of creating a ``PeerArena`` (several ranks emulated by one process on one GPU;
        the closing all-reduce is then left to the caller)."""
        import torch

        self.fb, self.world, self.me, self.local = fb, world, me, False
        self.names = list(requests)
        self.frames: Dict[str, TensorFrame] = {}
        self.device = next(l.device for ls in fb.rank_loaders.values() for l in ls)
        if self.device.is_cpu:
            raise Exception("the peer transport needs CUDA devices")
        self.chunks: List[_Chunk] = []
        self.chunk_base: List[List[int]] = []      # [chunk][rank] -> offset in that rank's arena
        total = [0] * world
        for names in cut_into_chunks(fb, requests, world, chunk_bytes or (1 << 62)):
            lay = BatchLayout(world)
            for name in names:
                rank, lidx = fb._get_rank_lidx(name)
                frame = fb.rank_loaders[rank][lidx].metadata.tensors[name]
                self.frames[name] = frame
                lay.add(name, frame, rank, requests[name])
            self.chunk_base.append(list(total))
            self.chunks.append(_Chunk(names, lay, total[me], lay.recv_total(me), 0))
            for r in range(world):
                total[r] += lay.recv_total(r)
        # every rank allocates for the neediest rank, so that all decide alike
        self.recv_need = max(total)
        self._own_arena = arena is None
        self.arena = PeerArena.for_group(fb.pg, max(total), self.device) if arena is None else arena
        self.recv = self.arena.view(total[me])
        self.send = None
        self.payload_bytes = 0
        self.egress_bytes = sum(ch.layout.region_bytes[me][d] for ch in self.chunks
                                for d in range(world) if d != me)
        self._flag = torch.zeros(1, dtype=torch.int32, device=self.device.as_str())
        self._side = None
        self.remote_ctas = peer_remote_ctas(world, self.device.index or 0)
        import os

        # order of the peer stores: "region" = one destination after the other, rotated per
        # owner; "interleave" = tensor by tensor to all destinations (see BatchLayout.fill_ops)
        self.order = "interleave" if os.environ.get("FST_B200_PEER_ORDER", "interleave") == "interleave" else True

    def _prepare(self, index: int) -> _Chunk:
        ch = self.chunks[index]
        if ch.launches is not None:
            return ch
        from . import _native as nat

        fb, lay, me = self.fb, ch.layout, self.me
        src_addr: Dict[str, int] = {}
        for name in ch.names:
            rank, lidx = fb._get_rank_lidx(name)
            if rank == me:
                loader = fb.rank_loaders[rank][lidx]
                tensors = loader.tensors          # completes a deferred read of the file
                if name not in tensors:
                    raise Exception(f"exchange: tensor {name} was not found, released? lidx={loader.lidx}")
                src_addr[name] = tensors[name].data_ptr()
        # region [me -> d]: d's arena, this chunk's part, at the offset where d expects owner `me`
        base = self.chunk_base[index]
        region = [self.arena.peer_base[d] + base[d] + lay.recv_offset(d, me) for d in range(self.world)]
        mine = {n: self.frames[n] for n in src_addr}
        ops = lay.fill_ops(me, mine, src_addr, region, rotate=self.order) if mine else []
        ch.payload = sum(o[2] * o[3] for o in ops)
        lo, hi = self.arena.address, self.arena.address + self.arena.nbytes
        own = [o for o in ops if lo <= o[1] < hi]
        remote = [o for o in ops if not (lo <= o[1] < hi)]
        if self.remote_ctas > 0 and own and remote:
            # two launches side by side: the peer stores on a grid small enough to leave most of
            # the SMs to this rank's own region (see run)
            ch.launches = [(nat.pack_ops(remote), len(remote), "remote"), (nat.pack_ops(own), len(own), "own")]
        else:
            ch.launches = [(nat.pack_ops(ops), len(ops), "all")] if ops else []
        return ch

    def run(self, timing: Optional[list] = None, after_chunk=None) -> None:
        import torch
        import torch.distributed as dist

        from . import _native as nat

        cur = torch.cuda.current_stream()
        payload = 0
        for index in range(len(self.chunks)):
            ch = self._prepare(index)
            payload += ch.payload
            split = len(ch.launches) == 2
            if split:
                if self._side is None:
                    self._side = torch.cuda.Stream()
                self._side.wait_stream(cur)          # the images are ready on the caller's stream
            for packed, n, kind in ch.launches:
                stream = self._side if kind == "own" and split else cur
                if timing is not None:
                    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    a.record(stream)
                nat.check(nat.lib.fst_gather_limited(packed.pointer, n, 0, 0, 0, 0, int(stream.cuda_stream),
                                                     self.remote_ctas if kind == "remote" else 0),
                          "fst_gather")
                if timing is not None:
                    b.record(stream)
                    timing.append((a, b))
            if split:
                cur.wait_stream(self._side)          # before the image is released or reused
            if after_chunk is not None:
                after_chunk(ch.names)
        self.payload_bytes = payload
        # every rank's kernels are complete (a kernel's peer stores are visible when it completes)
        if self._own_arena:
            dist.all_reduce(self._flag, group=self.fb.pg.real_pg)

    def _view(self, slot: Slot, off: int):
        from .frameworks._torch import TorchTensor, dtype_convert

        frame = self.frames[slot.name]
        native = self.fb.framework.get_native_shape(frame.dtype, slot.shape)
        t = self.recv[off: off + slot.nbytes].view(dtype_convert[frame.dtype]).reshape(native)
        return TorchTensor(self.device, frame.dtype, t)

    def results(self):
        out = {}
        for ch in self.chunks:
            for slot, off in ch.layout.received(self.me):
                out[slot.name] = self._view(slot, ch.recv_base + off)
        return out

    def close(self) -> None:
        """Collective: the peers let go of each other's arenas (the results stay valid)."""
        if self._own_arena:
            self.arena.close_peers()

    def finish(self) -> None:
        self.close()
