"""Makes ``import fastsafetensors`` resolve to this package.

``install()`` enters this package and its submodules into ``sys.modules`` under upstream's module
names (``fastsafetensors``, ``fastsafetensors.cpp``, ``fastsafetensors.common``,
``fastsafetensors.copier.nogds`` ...), so that code written against upstream (vLLM's
``fastsafetensors`` load format, TGIS-style weight loaders) runs on the B200 loader without
edits.  Call it before the first such import.
"""

from __future__ import annotations

import importlib
import sys

_PREFIX = "fastsafetensors"
_TARGET = "fastsafetensors_b200"
_SUBMODULES = (
    "", ".cpp", ".common", ".st_types", ".loader", ".file_buffer", ".tensor_factory",
    ".frameworks", ".frameworks._torch", ".copier", ".copier.base", ".copier.registry",
    ".copier.nogds", ".copier.gds", ".parallel_loader", ".config", ".auto_loader",
)


def install() -> None:
    """Idempotent.  Modules of an upstream installation that are already imported are replaced."""
    for sub in _SUBMODULES:
        try:
            module = importlib.import_module(_TARGET + sub)
        except ImportError:
            continue
        sys.modules[_PREFIX + sub] = module
