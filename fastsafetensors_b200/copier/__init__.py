"""Copier layer: the registry and the one copier this build has (see ``b200.py``)."""

from .b200 import B200FileCopier, new_b200_file_copier
from .base import CopierInterface, DummyDeviceBuffer
from .registry import (
    CopierConstructFunc,
    CopierType,
    create_copier_constructor,
    register_copier_constructor,
)

# upstream's class names, for callers that import them
NoGdsFileCopier = B200FileCopier
GdsFileCopier = B200FileCopier
