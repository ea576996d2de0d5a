"""B200-native safetensors weight loader with the API of fastsafetensors.

``SafeTensorsFileLoader`` / ``fastsafe_open`` read ``.safetensors`` files through a native
multi-threaded reader into HBM, and ``FilesBufferOnDevice`` hands out whole, sharded, column-
packed or pushed tensors, packing shards with one CUDA gather launch per request.  The native
layer is ``libfst_b200.so`` (C ABI in ``include/fst_b200.h``); importing this package fails if it
has not been built.
"""

__version__ = "0.1.0"

from .auto_loader import AutoLoader
from .common import SafeTensorsMetadata, SingleGroup, TensorFrame, get_device_numa_node
from .config import LoaderConfig, load_config
from .file_buffer import FilesBufferOnDevice
from .loader import BaseSafeTensorsFileLoader, SafeTensorsFileLoader, fastsafe_open
from .parallel_loader import ParallelLoader, PipelineParallel
from .st_types import Device, DeviceType, DType

__all__ = [
    "AutoLoader", "LoaderConfig", "load_config", "BaseSafeTensorsFileLoader", "Device", "DeviceType", "DType", "FilesBufferOnDevice",
    "ParallelLoader", "PipelineParallel", "SafeTensorsFileLoader", "SafeTensorsMetadata", "SingleGroup", "TensorFrame",
    "fastsafe_open", "get_device_numa_node",
]
