"""Upstream's module name for the cuFile copier; here it is the B200 copier."""

from .b200 import B200FileCopier as GdsFileCopier  # noqa: F401
from .b200 import new_b200_file_copier as new_gds_file_copier  # noqa: F401


def init_gds() -> None:
    """Upstream opens the cuFile driver here; this build has nothing to open."""
