"""Loader entry points: ``SafeTensorsFileLoader`` and ``fastsafe_open``.

Source-compatible with upstream ``fastsafetensors/loader.py`` (constructor arguments, methods
``add_filenames``, ``copy_files_to_device``, ``get_keys``, ``get_shape``, ``reset``, ``close``;
attributes ``meta``, ``frames``, ``pg``, ``device``, ``framework``), which is the call sequence
vLLM's ``fastsafetensors`` load format drives.  Whatever the ``nogds`` flag says, files are read
by the B200 copier (``copier/b200.py``); the flag only picks the registry name.
"""

from __future__ import annotations

import math
from collections import OrderedDict
from typing import Any, Dict, List, Mapping, Optional, Tuple, Union

from . import cpp as fstcpp
from .common import SafeTensorsMetadata, TensorFrame, get_device_numa_node, init_logger
from .copier import CopierConstructFunc, CopierType, create_copier_constructor
from .file_buffer import FilesBufferOnDevice
from .frameworks import TensorBase, get_framework_op
from .st_types import Device, DeviceType, DType
from .tensor_factory import LazyTensorFactory

logger = init_logger(__name__)

DEFAULT_MAX_COPY_BLOCK = 16 * 1024 * 1024 * 1024
_numa_pinned = False


class BaseSafeTensorsFileLoader:
    """Registers files per owner rank and copies them to device buffers.

    Args:
        pg: process group (``torch.distributed.ProcessGroup``), ``SingleGroup()`` or None.
        device: a ``Device`` naming where tensors go.
        copier_type: registry name of the copier factory.
        set_numa: bind the process to the NUMA node of the device (once per process).
        disable_cache: do not keep shuffled tensors for repeated requests.
        framework: ``"pytorch"`` / ``"pt"`` / ``"torch"``.
        **kwargs: passed to the copier factory (``bbuf_size_kb``, ``max_threads``, ...).
    """

    @classmethod
    def process_extension_config(cls, ext_config: Mapping[str, Any], **kwargs: Any) -> Dict[str, Any]:
        return dict(ext_config)

    def __init__(self, pg: Optional[Any], device: Device, copier_type: CopierType,
                 set_numa: bool = True, disable_cache: bool = True, framework="pytorch", **kwargs):
        self.framework = get_framework_op(framework)
        self.pg = self.framework.get_process_group(pg)
        self.device = device
        self.meta: Dict[str, Tuple[SafeTensorsMetadata, int]] = {}
        self.frames: Dict[str, TensorFrame] = OrderedDict()
        self.disable_cache = disable_cache
        numa_node = self.init_numa(set_numa)
        if numa_node is not None:
            kwargs.setdefault("numa_node", numa_node)
        self.copier_constructor: CopierConstructFunc = create_copier_constructor(
            copier_type=copier_type, device=device, framework=self.framework, **kwargs
        )

    def init_numa(self, set_numa: bool = True) -> Optional[int]:
        """Bind this process to the device's NUMA node once (loader.py:75-81) and return it so
        the reader can bind its workers and ring too."""
        global _numa_pinned
        if not set_numa or self.device.type == DeviceType.CPU:
            return None
        node = get_device_numa_node(self.device.index if self.device.index is not None else 0)
        if node is not None and not _numa_pinned:
            fstcpp.set_numa_node(node)
        _numa_pinned = True
        return node

    def reset(self) -> None:
        self.frames = OrderedDict()
        self.meta = {}

    def close(self) -> None:
        self.reset()
        ctor = getattr(self, "copier_constructor", None)
        if ctor is not None:
            reader = getattr(ctor, "reader", None)
            if reader is not None:
                reader.close()
            del self.copier_constructor

    def get_keys(self) -> List[str]:
        return list(self.frames.keys())

    def get_shape(self, tensor_name: str) -> List[int]:
        return self.frames[tensor_name].shape

    def add_filenames(self, filenames: Dict[int, List[str]]) -> None:
        """Register ``{owner rank: [paths]}``.  Files are interleaved across ranks (first file
        of every rank, then the second, ...) so that registration order spreads memory use
        (loader.py:97-119).  Every rank parses every header."""
        depth = max((len(v) for v in filenames.values()), default=0)
        for i in range(depth):
            for rank, paths in filenames.items():
                if i < len(paths):
                    path = paths[i]
                    metadata = SafeTensorsMetadata.from_file(path, self.framework)
                    self.meta[path] = (metadata, rank)
                    self.frames.update(metadata.tensors)

    def copy_files_to_device(self, dtype: DType = DType.AUTO, use_buf_register: bool = True,
                             max_copy_block_size: int = DEFAULT_MAX_COPY_BLOCK,
                             wait: bool = True) -> FilesBufferOnDevice:
        """Start the reads of all files this rank owns, wait for them, and return the buffer
        object through which tensors are instantiated.  Files are taken in sorted path order;
        a file's 1-based position is its id in send/recv tags (loader.py:121-168).

        ``wait=False`` (not in upstream) returns as soon as the reads are queued.  Each file is
        then waited for by the first access to one of its tensors, so a caller that works
        through the files in order -- ``FilesBufferOnDevice.exchange`` / ``as_dict`` /
        ``shard_locally`` do -- packs and ships file k while the native reader is still filling
        files k+1, k+2, ...; a failed read surfaces at that access instead of here."""
        self.framework.set_device(self.device)
        me = self.pg.rank()
        factories: Dict[int, List[LazyTensorFactory]] = {r: [] for r in range(self.pg.size())}
        idx_bits = math.ceil(math.log2(len(self.meta) + 1))
        mine: List[LazyTensorFactory] = []
        for lidx, path in enumerate(sorted(self.meta), start=1):
            meta, rank = self.meta[path]
            is_mine = rank == me
            copier = self.copier_constructor(meta, self.device, self.framework) if is_mine else None
            factory = LazyTensorFactory(meta, self.device, rank, is_mine, idx_bits, lidx, copier,
                                        self.framework, disable_cache=self.disable_cache)
            factory.submit_io(use_buf_register, max_copy_block_size)
            factories[rank].append(factory)
            if is_mine:
                mine.append(factory)
        error: Optional[BaseException] = None
        for factory in mine:  # drain every request even if one fails
            if not wait:
                factory.defer_wait(dtype=dtype, noalign=False)
                continue
            try:
                factory.wait_io(dtype=dtype, noalign=False)
            except Exception as e:  # noqa: BLE001
                error = error or e
        if error is not None:
            for factory in mine:
                factory.free_dev_ptrs()
            raise error
        try:
            return FilesBufferOnDevice(factories, pg=self.pg, framework=self.framework)
        except Exception:
            for factory in mine:
                factory.free_dev_ptrs()
            raise


class SafeTensorsFileLoader(BaseSafeTensorsFileLoader):
    """Load ``.safetensors`` files lazily.

    Args:
        pg: process group; None or ``SingleGroup()`` for one process.
        device: target device, ``str`` or ``torch.device``.
        bbuf_size_kb: lower bound of the pinned ring size in KiB.
        max_threads: reader worker threads.
        nogds: kept for compatibility; both settings use the same copier here.
        set_numa / disable_cache / debug_log / framework: as upstream.
        **kwargs: copier options (``io_mode``, ``slot_kb``, ``copy_streams``, ...).
    """

    @classmethod
    def process_extension_config(cls, ext_config: Mapping[str, Any], **kwargs: Any) -> Dict[str, Any]:
        out = dict(ext_config)
        out["nogds"] = out.pop("copier_type", "gds") != "gds"
        return out

    def __init__(self, pg: Optional[Any], device: Any = "cpu", bbuf_size_kb: int = 16 * 1024,
                 max_threads: int = 16, nogds: bool = False, set_numa: bool = True,
                 disable_cache: bool = True, debug_log: bool = False, framework="pytorch", **kwargs):
        fw = get_framework_op(framework)
        dev = fw.get_device(device, fw.get_process_group(pg))
        fstcpp.set_debug_log(debug_log)
        super().__init__(pg, dev, "nogds" if nogds else "gds", set_numa, disable_cache, framework,
                         bbuf_size_kb=bbuf_size_kb, max_threads=max_threads, **kwargs)


class fastsafe_open:
    """Context manager over one or more files, in the manner of ``safetensors.safe_open``.

    Args:
        filenames: a path, a list of paths, or ``{rank: [paths]}``.
        framework: ``"pt"`` / ``"pytorch"``.
        pg, device, nogds, debug_log, max_copy_block_size: as for the loader.

    Tensors are valid while the context is open; clone them to keep them longer.
    """

    def __init__(self, filenames: Union[str, List[str], Dict[int, List[str]]], framework: str = "pt",
                 pg: Optional[Any] = None, device: Any = "cpu", nogds: bool = False,
                 debug_log: bool = False, max_copy_block_size: int = DEFAULT_MAX_COPY_BLOCK):
        self.loader = SafeTensorsFileLoader(pg, device, nogds=nogds, debug_log=debug_log,
                                            framework=framework)
        if isinstance(filenames, str):
            file_dict: Dict[int, List[str]] = {0: [filenames]}
        elif isinstance(filenames, list):
            file_dict = {0: filenames}
        elif isinstance(filenames, dict):
            file_dict = filenames
        else:
            file_dict = {}
        self.loader.add_filenames(file_dict)
        self.fb = self.loader.copy_files_to_device(max_copy_block_size=max_copy_block_size)

    def metadata(self) -> Dict[str, Dict[str, str]]:
        return {path: meta.metadata for path, (meta, _) in self.loader.meta.items()}

    def keys(self) -> List[str]:
        return list(self.fb.key_to_rank_lidx.keys())

    def get_tensor_wrapped(self, name: str) -> TensorBase:
        return self.fb.get_tensor_wrapped(name)

    def get_tensor(self, name: str) -> Any:
        return self.get_tensor_wrapped(name).get_raw()

    def __enter__(self):
        return self

    def __exit__(self, exc_type, exc_value, tb):
        if self.fb:
            self.fb.close()
        if self.loader:
            self.loader.close()
