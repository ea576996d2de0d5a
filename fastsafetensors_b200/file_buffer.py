"""``FilesBufferOnDevice``: name-addressed access to the tensors of a batch of loaded files.

Public surface of upstream ``fastsafetensors/file_buffer.py``: ``get_tensor``, ``get_sharded``,
``push_tensor``, ``get_multi_cols``, ``as_dict`` and their ``*_wrapped`` forms, ``get_filename``,
``get_shape``, ``close``, and the attributes ``key_to_rank_lidx``, ``rank_loaders``,
``auto_mem_delete`` that callers read.  In multi-rank use every rank must call these methods in
the same order (they end in collectives).
"""

from __future__ import annotations

import os
from collections import OrderedDict
from typing import Any, Dict, List, Optional, Tuple

from .common import init_logger
from .frameworks import ProcessGroupBase, TensorBase
from .st_types import Device, DType
from .tensor_factory import LazyTensorFactory

logger = init_logger(__name__)


# "auto" picks the peer transport for groups of up to this many ranks (one NVSwitch machine): on
# B200 it measured 13.9 ms against 31 ms per step for the NCCL all-to-all at two ranks and 14 ms
# against 48 ms at four (38 GB checkpoint); larger groups span machines, where peer mapping is
# refused anyway.
PEER_AUTO_MAX_WORLD = 8


def resolve_transport(transport: Optional[str], world: int, device) -> str:
    """``"nccl"``, ``"peer"`` or ``"auto"`` (= try peer, fall back) for an exchange among
    ``world`` ranks on ``device``; ``None`` reads ``FST_B200_TRANSPORT`` (default ``auto``)."""
    if transport is None:
        transport = os.environ.get("FST_B200_TRANSPORT", "auto")
    if transport not in ("nccl", "peer", "auto"):
        raise ValueError(f"transport must be 'nccl', 'peer' or 'auto', got {transport!r}")
    if device.is_cpu:
        if transport == "peer":
            raise Exception("the peer transport needs CUDA devices")
        return "nccl"
    if transport == "auto" and world > PEER_AUTO_MAX_WORLD:
        return "nccl"
    return transport


class FilesBufferOnDevice:
    def __init__(self, rank_loaders: Dict[int, List[LazyTensorFactory]], pg: ProcessGroupBase,
                 framework, auto_mem_delete: bool = True):
        self.framework = framework
        self.rank_loaders = rank_loaders
        self.pg = pg
        self.key_to_rank_lidx: Dict[str, Tuple[int, int]] = {}
        # per file: names already handed out; a file image is dropped once all were
        self.instantiated: Dict[int, Dict[int, Dict[str, bool]]] = {}
        for rank, loaders in rank_loaders.items():
            self.instantiated[rank] = {}
            for lidx, loader in enumerate(loaders):
                self.instantiated[rank][lidx] = {}
                for key in loader.metadata.tensors:
                    if key in self.key_to_rank_lidx:
                        raise Exception(f"FilesBufferOnDevice: key {key} must be unique among files")
                    self.key_to_rank_lidx[key] = (rank, lidx)
        # with one rank results alias the images, so the images must stay
        self.auto_mem_delete = auto_mem_delete and pg.size() > 1

    def close(self) -> None:
        """Drop the file images.  Tensors obtained with one rank are views of them."""
        for loaders in self.rank_loaders.values():
            for loader in loaders:
                loader.free_dev_ptrs()
        self.rank_loaders = {}

    def replicate_all(self) -> None:
        """Give every rank every file image of this batch: one broadcast per file, after which
        ``get_tensor`` returns views without further collectives.  This is the bulk form of
        "``get_tensor`` for every key", the access pattern of vLLM's loader and of
        ``PipelineParallel``.  Collective: all ranks call it at the same point."""
        if self.pg.size() == 1:
            return
        for rank in sorted(self.rank_loaders):
            for loader in self.rank_loaders[rank]:
                loader.replicate(self.pg)

    def get_filename(self, tensor_name: str) -> str:
        if tensor_name not in self.key_to_rank_lidx:
            return ""
        rank, lidx = self.key_to_rank_lidx[tensor_name]
        return self.rank_loaders[rank][lidx].metadata.src

    def get_shape(self, tensor_name: str) -> List[int]:
        rank, lidx = self._get_rank_lidx(tensor_name)
        return self.rank_loaders[rank][lidx].metadata.tensors[tensor_name].shape

    def _get_rank_lidx(self, tensor_name: str) -> Tuple[int, int]:
        try:
            return self.key_to_rank_lidx[tensor_name]
        except KeyError:
            raise ValueError(f"_get_rank: key {tensor_name} was not found in files") from None

    def _mark(self, rank: int, lidx: int, tensor_name: str) -> None:
        """Record that ``tensor_name`` was handed out; free its file image after the last one."""
        if not self.auto_mem_delete:
            return
        loader = self.rank_loaders[rank][lidx]
        seen = self.instantiated[rank][lidx]
        seen[tensor_name] = True
        if len(seen) == len(loader.metadata.tensors):
            if self.pg.rank() == rank:
                logger.debug("free_dev_ptrs: lidx=%d, src=%s", lidx, loader.metadata.src)
            loader.free_dev_ptrs()

    def _get_tensor(self, rank: int, lidx: int, tensor_name: str, ret: TensorBase,
                    device: Optional[Device], dtype: DType) -> TensorBase:
        self._mark(rank, lidx, tensor_name)
        return ret.to(device=device, dtype=dtype)

    # ------------------------------------------------------------------ one tensor
    def get_sharded_wrapped(self, tensor_name: str, dim: int, device: Optional[Device] = None,
                            dtype: DType = DType.AUTO) -> TensorBase:
        rank, lidx = self._get_rank_lidx(tensor_name)
        t = self.rank_loaders[rank][lidx].shuffle(self.pg, tensor_name, dim)
        return self._get_tensor(rank, lidx, tensor_name, t, device, dtype)

    def get_sharded(self, tensor_name: str, dim: int, device: Optional[Device] = None,
                    dtype: DType = DType.AUTO) -> Any:
        """This rank's block of ``tensor_name`` on ``dim`` (``dim == -1``: the whole tensor)."""
        return self.get_sharded_wrapped(tensor_name, dim, device, dtype).get_raw()

    def get_tensor_wrapped(self, tensor_name: str, device: Optional[Device] = None,
                           dtype: DType = DType.AUTO) -> TensorBase:
        return self.get_sharded_wrapped(tensor_name, -1, device, dtype)

    def get_tensor(self, tensor_name: str, device: Optional[Device] = None,
                   dtype: DType = DType.AUTO) -> Any:
        """The whole tensor on every rank (broadcast from the rank that read its file)."""
        return self.get_tensor_wrapped(tensor_name, device, dtype).get_raw()

    def push_tensor(self, tensor_name: str, dst_rank: int, device: Optional[Device] = None,
                    dtype: DType = DType.AUTO) -> Optional[Any]:
        """The whole tensor on ``dst_rank`` only; None elsewhere."""
        rank, lidx = self._get_rank_lidx(tensor_name)
        t = self.rank_loaders[rank][lidx].push(self.pg, tensor_name, dst_rank, rank)
        if t is None:
            self._mark(rank, lidx, tensor_name)
            return None
        return self._get_tensor(rank, lidx, tensor_name, t, device, dtype).get_raw()

    # ------------------------------------------------------------------ column groups
    def get_multi_cols(self, tensor_names: List[str], dim: int, device: Optional[Device] = None,
                       dtype: DType = DType.AUTO) -> TensorBase:
        """This rank's shards of ``tensor_names`` concatenated on ``dim`` (a wrapped tensor, as
        upstream returns).  Names are grouped by file; groups are emitted in (owner, file)
        order, names inside a group in the order given (file_buffer.py:204-221)."""
        groups: Dict[Tuple[int, int], List[str]] = {}
        for name in tensor_names:
            groups.setdefault(self._get_rank_lidx(name), []).append(name)
        parts: List[TensorBase] = []
        for (rank, lidx) in sorted(groups):
            parts.append(self.rank_loaders[rank][lidx].shuffle_multi_cols(self.pg, groups[(rank, lidx)], dim))
        ret = parts[0] if len(parts) == 1 else self.framework.concat_tensors(parts, dim=dim)
        for name in tensor_names:
            self._mark(*self.key_to_rank_lidx[name], name)
        return ret.to(device=device, dtype=dtype)

    # ------------------------------------------------------------------ many tensors
    def as_dict(self, tensor_shard_dim: "OrderedDict[str, int]") -> Dict[str, TensorBase]:
        """``{name: wrapped tensor}`` for ``{name: dim}`` (``-1`` = replicate).  With more than
        one rank the whole request is served by the batched exchange (see ``exchange``)."""
        requests = OrderedDict(
            (name, ("replicate",) if dim == -1 else ("shard", dim))
            for name, dim in tensor_shard_dim.items()
        )
        return self.exchange(requests)

    def exchange(self, requests: "OrderedDict[str, Tuple]", max_batch_bytes: int = 8 << 30,
                 transport: Optional[str] = None) -> Dict[str, TensorBase]:
        """Serve many requests at once: ``{name: ("shard", dim) | ("replicate",) | ("push", r)}``.

        The requests are taken round by round (round j = the j-th file of every owner) and cut
        into chunks of at most ``min(max_batch_bytes, FST_B200_EXCHANGE_CHUNK_MB)`` outgoing bytes
        per owner.  Per chunk every owner packs what it has to send with one gather launch and
        all ranks meet in ONE ``all_to_all_single``, started asynchronously so that the next
        chunk is packed (and, after ``copy_files_to_device(wait=False)``, still being read)
        while this one travels; upstream issues a collective and a device synchronisation per
        tensor (tensor_factory.py:143,186).  Results are views of one receive buffer.  A file
        image is released as soon as its last tensor has been packed.  For a pushed tensor only
        the destination rank gets an entry.  Every rank must pass the same requests in the same
        order.

        ``transport``: ``"nccl"`` packs into a send buffer and exchanges with
        ``all_to_all_single``; ``"peer"`` (CUDA devices of one machine) lets the gather kernel
        store every shard straight into the destination rank's receive arena over NVLink (the
        results are views of that arena), and raises ``PeerArenaUnavailable`` on every rank if
        the ranks cannot map each other's memory; ``"auto"`` uses ``"peer"`` for groups of up to
        ``PEER_AUTO_MAX_WORLD`` ranks and falls back to ``"nccl"``, on all ranks together, where
        peer mapping is refused.
        Default: the ``FST_B200_TRANSPORT`` environment variable, else ``"auto"``.
        """
        from .batch import PeerArena, PeerArenaUnavailable, PeerShardExchange, ShardExchange, default_chunk_bytes

        world, me = self.pg.size(), self.pg.rank()
        out: Dict[str, TensorBase] = {}
        if world == 1:
            for name in requests:
                rank, lidx = self._get_rank_lidx(name)
                out[name] = self.rank_loaders[rank][lidx].tensors[name]
            return out
        device = next(l.device for ls in self.rank_loaders.values() for l in ls)
        transport = resolve_transport(transport, world, device)
        fall_back = transport == "auto"
        if fall_back and PeerArena.known_unusable(self.pg, device):
            transport = "nccl"      # tried before on this group: all ranks know, nobody asks again

        def release(names: List[str]) -> None:
            for name in names:
                self._mark(*self.key_to_rank_lidx[name], name)

        if transport in ("peer", "auto"):
            try:
                ex = PeerShardExchange(self, requests, world, me,
                                       chunk_bytes=max_batch_bytes if max_batch_bytes < (8 << 30) else None)
            except PeerArenaUnavailable as e:
                # raised by all ranks at the same call, so all take the same branch
                if not fall_back:
                    raise
                logger.warning("exchange: %s; using the NCCL all-to-all", e)
            else:
                ex.run(after_chunk=release)
                out.update(ex.results())
                ex.close()
                return out
        ex = ShardExchange(self, requests, world, me, local=False,
                           chunk_bytes=min(max_batch_bytes, default_chunk_bytes()))
        ex.run(after_chunk=release)
        out.update(ex.results())
        return out

    def shard_locally(self, requests: "OrderedDict[str, Tuple]", world_size: int) -> List[Dict[str, TensorBase]]:
        """Single-process form of ``exchange``: this process (which must own every file of the
        requests, i.e. was opened with one rank) produces what each of ``world_size``
        tensor-parallel ranks would receive, with one gather launch.  Returns one
        ``{name: wrapped tensor}`` per destination rank; the tensors are views of one buffer."""
        from .batch import ShardExchange

        if self.pg.size() != 1:
            raise Exception("shard_locally needs a single-rank loader (it owns every file)")
        ex = ShardExchange(self, requests, world_size, 0, local=True)
        ex.run()
        return ex.results()
