"""Per-file tensor factory: owns one file image and turns it into replicated, sharded,
column-packed or pushed tensors.

Same role and method names as upstream ``fastsafetensors/tensor_factory.py``
(``LazyTensorFactory``: ``submit_io``, ``wait_io``, ``shuffle``, ``shuffle_multi_cols``,
``push``, ``free_dev_ptrs``).  What differs is how the owner rank prepares what it sends:

* upstream runs, per tensor, ``world_size`` slice + ``.contiguous()`` launches
  (``tensor_factory.py:168-175``) or ``world_size`` ``torch.cat`` launches (``:240-246``);
* here the owner describes all ``world_size`` shards (and all members of a column group) as
  strided byte copies and packs them with ONE launch of the gather kernel into a buffer laid
  out ``[rank][shard bytes]``, whose rows are then scattered.  Shards that are already
  contiguous in the file image (a split on the outermost dimension) are scattered straight
  from the image without any copy.
"""

from __future__ import annotations

import os
from typing import Dict, List, Optional

from . import _native as nat
from . import shard_plan
from .common import SafeTensorsMetadata, init_logger
from .copier.base import CopierInterface, DummyDeviceBuffer
from .frameworks import ProcessGroupBase, TensorBase
from .frameworks._torch import TorchTensor
from .st_types import Device, DType

logger = init_logger(__name__)
HOST_GATHER_THREADS = 8
# fraction of a file that may be broadcast tensor by tensor before the whole image is broadcast
# instead (0 disables the switch); see LazyTensorFactory.shuffle
REPLICATE_FILE_AFTER = float(os.environ.get("FST_B200_REPLICATE_FILE_AFTER", "0.25"))


class LazyTensorFactory:
    def __init__(self, metadata: SafeTensorsMetadata, device: Device, rank: int, local_rank: bool,
                 factory_idx_bits: int, lidx: int, copier: Optional[CopierInterface], framework,
                 disable_cache: bool = True):
        self.framework = framework
        self.metadata = metadata
        self.device = device
        self.copier: Optional[CopierInterface] = copier if local_rank else None
        self._tensors: Dict[str, TensorBase] = {}
        self._deferred: Optional[tuple] = None   # (dtype, noalign) of a wait_io still to be done
        self.shuffled: Dict[str, TensorBase] = {}
        self.gbuf = None
        self.rank = rank                    # owner of the file
        self.factory_idx_bits = factory_idx_bits
        self.lidx = lidx                    # 1-based index of the file among all files
        self.next_tag = 1
        self.disable_cache = disable_cache
        self.replicated = False             # every rank holds the image (see replicate)
        self.converted = False              # tensors were narrowed in place at load time
        self.broadcast_bytes = 0            # bytes handed out one tensor at a time with dim -1

    # ---------------------------------------------------------------- file -> image
    def submit_io(self, use_buf_register: bool, max_copy_block_size: int) -> None:
        if self.copier is not None:
            self.gbuf = self.copier.submit_io(use_buf_register, max_copy_block_size)
            logger.debug("submit_io: new buf, addr=0x%x", self.gbuf.get_base_address())

    def wait_io(self, dtype: DType = DType.AUTO, noalign: bool = False) -> None:
        self._deferred = None
        if self.copier is not None and self.gbuf is not None:
            copier, self.copier = self.copier, None
            try:
                self._tensors = copier.wait_io(self.gbuf, dtype=dtype, noalign=noalign)
            except Exception:
                self.free_dev_ptrs()
                raise
            self.converted = dtype != DType.AUTO

    def defer_wait(self, dtype: DType = DType.AUTO, noalign: bool = False) -> None:
        """Leave the read running: ``wait_io`` is done by the first access to ``tensors``
        (``copy_files_to_device(wait=False)``), so that whoever consumes the files one after the
        other overlaps its work on file k with the reads of files k+1, k+2, ..."""
        if self.copier is not None and self.gbuf is not None:
            self._deferred = (dtype, noalign)

    @property
    def pending(self) -> bool:
        """True while this rank's read of the file has been started but not yet waited for."""
        return self._deferred is not None

    def ensure_loaded(self) -> None:
        if self._deferred is not None:
            dtype, noalign = self._deferred
            self.wait_io(dtype=dtype, noalign=noalign)

    @property
    def tensors(self) -> Dict[str, TensorBase]:
        """Tensors over this rank's image of the file (empty on ranks that hold no image).
        Completes a deferred read first."""
        if self._deferred is not None:
            self.ensure_loaded()
        return self._tensors

    @tensors.setter
    def tensors(self, value: Dict[str, TensorBase]) -> None:
        self._tensors = value

    def free_dev_ptrs(self) -> None:
        if self._deferred is not None:
            # the reader is still writing into the image: drain the request before the memory
            # goes back to the allocator (errors of a read nobody wants any more are dropped)
            self._deferred = None
            copier, self.copier = self.copier, None
            if copier is not None and self.gbuf is not None:
                try:
                    copier.drain()
                except Exception:  # noqa: BLE001
                    pass
        self._tensors = {}
        if self.gbuf is not None and not isinstance(self.gbuf, DummyDeviceBuffer):
            logger.debug("free_dev_ptrs: delete buf, addr=0x%x", self.gbuf.get_base_address())
            self.framework.free_tensor_memory(self.gbuf, self.device)
            self.gbuf = None

    def replicate(self, pg: ProcessGroupBase) -> bool:
        """Broadcast the whole file image from its owner so that every rank can instantiate every
        tensor of the file as a view: one collective per file instead of one per tensor.
        Collective: every rank must call it, in the same file order.  Returns False (and does
        nothing) when the image cannot be shared as it is."""
        if pg.size() == 1 or self.replicated:
            return True
        if self.converted:   # in-place narrowing changed the owner's layout only
            return False
        owner = self.rank == pg.rank()
        total = self.metadata.size_bytes - self.metadata.header_length
        if owner:
            self.ensure_loaded()
        if owner and self.gbuf is None:
            raise Exception(f"replicate: the image of {self.metadata.src} was already released")
        if not owner:
            self.gbuf = self.framework.alloc_tensor_memory(total, self.device)
        if total:
            pg.broadcast(TorchTensor(self.device, DType.U8, self.gbuf.owner[:total]), self.rank)
        if not owner:
            self.tensors = self.metadata.get_tensors(self.gbuf, self.device, self.metadata.header_length)
        self.replicated = True
        return True

    # ---------------------------------------------------------------- helpers
    def _owned(self, what: str, tensor_name: str) -> TensorBase:
        if tensor_name not in self.tensors:
            raise Exception(f"{what}: tensor {tensor_name} was not found, released? lidx={self.lidx}")
        return self.tensors[tensor_name]

    def _bytes_buffer(self, nbytes: int):
        import torch

        return torch.empty(nbytes, dtype=torch.uint8,
                           device=self.device.as_str() if not self.device.is_cpu else "cpu")

    def _run_ops(self, ops: List[shard_plan.Op], src_span, dst_span) -> None:
        """One gather launch on torch's current stream (device) or the host gather (cpu)."""
        if self.device.is_cpu:
            nat.gather_host(ops, threads=HOST_GATHER_THREADS)
        else:
            nat.gather(ops, self.framework.current_stream(self.device), src_span, dst_span)

    def _image_span(self):
        if self.gbuf is None:
            return (0, 0)
        return (self.gbuf.get_base_address(), self.gbuf.get_length())

    def _rows_of(self, packed, world_size: int) -> List[TorchTensor]:
        per_rank = packed.numel() // world_size
        return [TorchTensor(self.device, DType.U8, packed[r * per_rank:(r + 1) * per_rank])
                for r in range(world_size)]

    # ---------------------------------------------------------------- whole tensor to one rank
    def push(self, pg: ProcessGroupBase, tensor_name: str, dst_rank: int,
             src_rank: int) -> Optional[TensorBase]:
        """Send one whole tensor from the owner to ``dst_rank`` (tensor_factory.py:58-116).
        Ranks that are neither end return None."""
        if pg.size() == 1:
            return self.tensors[tensor_name]
        tag = (self.next_tag << self.factory_idx_bits) + self.lidx
        self.next_tag += 1
        me = pg.rank()
        if me != dst_rank and me != src_rank:
            return None
        if src_rank == dst_rank:
            return self._owned("push", tensor_name).clone().detach()
        frame = self.metadata.tensors[tensor_name]
        if me == src_rank:
            # straight out of the file image: the transport only reads it
            pg.send(self._owned("push", tensor_name), dst_rank, tag=tag)
            return None
        t = self.framework.get_empty_tensor(frame.shape, frame.dtype, self.device)
        pg.recv(t, src_rank, tag=tag)
        return t

    # ---------------------------------------------------------------- replicate / shard one tensor
    def shuffle(self, pg: ProcessGroupBase, tensor_name: str, dim: int) -> TensorBase:
        """``dim == -1``: every rank gets the whole tensor (broadcast from the owner);
        otherwise rank r gets block r of ``ceil(n/W)`` on ``dim`` (tensor_factory.py:118-192)."""
        world = pg.size()
        if world == 1:
            return self.tensors[tensor_name]  # alias of the file image
        if tensor_name in self.shuffled:
            return self.shuffled[tensor_name].clone().detach()
        frame = self.metadata.tensors[tensor_name]
        owner = self.rank == pg.rank()
        if dim == -1 and not self.replicated and not self.converted and REPLICATE_FILE_AFTER > 0:
            # A caller that asks for whole tensors one after the other (vLLM's loader asks for
            # every key) is better served by ONE broadcast of the file image than by a broadcast
            # per tensor.  Once a quarter of the file has gone out tensor by tensor, the rest
            # goes in one piece.  Every rank sees the same requests, so all switch together.
            self.broadcast_bytes += frame.data_offsets[1] - frame.data_offsets[0]
            image_bytes = self.metadata.size_bytes - self.metadata.header_length
            if self.broadcast_bytes >= image_bytes * REPLICATE_FILE_AFTER:
                self.replicate(pg)
        if dim == -1 and self.replicated:
            return self._owned("shuffle", tensor_name)   # view of this rank's copy of the image
        if dim == -1:
            if owner:
                dst = self._owned("shuffle", tensor_name).clone().detach()
            else:
                dst = self.framework.get_empty_tensor(frame.shape, frame.dtype, self.device)
            pg.broadcast(dst, self.rank)
        else:
            if not -1 < dim < len(frame.shape):
                raise IndexError(f"shuffle: dim {dim} is out of range for {tensor_name} {frame.shape}")
            shard_plan.check_even_split(tensor_name, frame.shape[dim], world)
            block = shard_plan.block_size(frame.shape[dim], world)
            new_shape = list(frame.shape)
            new_shape[dim] = block
            dst = self.framework.get_empty_tensor(new_shape, frame.dtype, self.device)
            chunks: List[TorchTensor] = []
            if owner:
                t = self._owned("shuffle", tensor_name)
                src = t.data_ptr()
                rows = shard_plan.slice_geometry(frame.shape, frame.dtype.bits, dim, 0, block)[0]
                if rows == 1:
                    # shards are contiguous in the image: scatter them as they lie
                    import torch

                    flat = t.get_raw().reshape(-1).view(torch.uint8)
                    chunks = self._rows_of(flat, world)
                else:
                    ops, shard_bytes = shard_plan.scatter_ops(
                        src, 0, frame.shape, frame.dtype.bits, dim, world)
                    packed = self._bytes_buffer(shard_bytes * world)
                    base = packed.data_ptr()
                    ops = [(o[0], o[1] + base) + o[2:] for o in ops]
                    self._run_ops(ops, self._span_of(t), (base, packed.numel()))
                    chunks = self._rows_of(packed, world)
            pg.scatter(dst, scatter_list=chunks, src=self.rank)
        if not self.disable_cache:
            self.shuffled[tensor_name] = dst
        return dst

    def _span_of(self, t: TensorBase):
        """Bounds handed to the gather's range check: the image, or the tensor's own bytes when
        it lives in the realign arena."""
        base, length = self._image_span()
        p = t.data_ptr()
        if base <= p < base + length:
            return (base, length)
        raw = t.get_raw()
        return (p, raw.numel() * raw.element_size())

    # ---------------------------------------------------------------- column groups
    def shuffle_multi_cols(self, pg: ProcessGroupBase, tensor_names: List[str], dim: int) -> TensorBase:
        """For each rank, concatenate on ``dim`` that rank's shard of every named tensor
        (fused QKV, gate/up) and deliver it (tensor_factory.py:194-259)."""
        world = pg.size()
        frames = [self.metadata.tensors[n] for n in tensor_names]
        dtype = frames[0].dtype
        shapes = [f.shape for f in frames]
        if world > 1:
            for n, f in zip(tensor_names, frames):
                shard_plan.check_even_split(n, f.shape[dim], world)
        owner = self.rank == pg.rank()
        srcs = [self._owned("shuffle_multi_cols", n).data_ptr() if owner else 0 for n in tensor_names]
        ops, per_rank, new_shape = shard_plan.multi_col_ops(srcs, 0, shapes, dtype.bits, dim, world)
        chunks: List[TorchTensor] = []
        if world == 1:
            dst = self.framework.get_empty_tensor(new_shape, dtype, self.device)
            base = dst.data_ptr()
            ops = [(o[0], o[1] + base) + o[2:] for o in ops]
            self._run_ops(ops, (0, 0), (base, per_rank))
            return dst
        if owner:
            packed = self._bytes_buffer(per_rank * world)
            base = packed.data_ptr()
            ops = [(o[0], o[1] + base) + o[2:] for o in ops]
            self._run_ops(ops, (0, 0), (base, packed.numel()))
            chunks = self._rows_of(packed, world)
        dst = self.framework.get_empty_tensor(new_shape, dtype, self.device)
        pg.scatter(dst, scatter_list=chunks, src=self.rank)
        return dst
