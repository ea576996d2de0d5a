"""Upstream's module name for the bounce-buffer copier; here it is the B200 copier."""

from .b200 import B200FileCopier as NoGdsFileCopier  # noqa: F401
from .b200 import new_b200_file_copier as new_nogds_file_copier  # noqa: F401


def load_library_func() -> None:
    """Upstream dlopen()s the CUDA runtime here; this build links it."""
