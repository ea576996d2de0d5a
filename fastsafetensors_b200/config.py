"""JSON / environment driven configuration of ``AutoLoader``.

Reads the same file format and follows the same discovery order as upstream
``fastsafetensors/config.py``: ``$FASTSAFETENSORS_CONFIG``, else ``./fastsafetensors.json``, else
defaults.  Top-level scalar keys and the members of the ``parallel`` and ``debug`` groups are core
settings; any other object-valued key (``base``, ...) is the settings section of the loader of
that name and is handed to it untouched (minus the settings common to all loaders).
"""

from __future__ import annotations

import json
import os
from dataclasses import dataclass, field, fields
from typing import Any, Dict

from .common import init_logger

logger = init_logger(__name__)

CONFIG_ENV_VAR = "FASTSAFETENSORS_CONFIG"
DEFAULT_CONFIG_PATH = "fastsafetensors.json"

_GROUPS = ("parallel", "debug")
_SHARED_WITH_EVERY_LOADER = ("framework", "debug_log", "set_numa", "disable_cache")


@dataclass
class LoaderConfig:
    loader: str = "base"
    framework: str = "pytorch"
    debug_log: bool = False
    set_numa: bool = True
    disable_cache: bool = True
    use_pipeline: bool = False
    max_concurrent_producers: int = 1
    queue_size: int = 0
    use_tqdm_on_load: bool = True
    _extensions: Dict[str, Dict[str, Any]] = field(default_factory=dict)

    def __post_init__(self) -> None:
        if self.max_concurrent_producers != 1:
            raise ValueError(
                f"max_concurrent_producers must be 1 (got {self.max_concurrent_producers}). "
                "Concurrent producers > 1 are not yet supported because broadcast "
                "batches must be processed in strict order across all ranks."
            )

    @classmethod
    def from_dict(cls, data: Dict[str, Any]) -> "LoaderConfig":
        known = {f.name for f in fields(cls) if not f.name.startswith("_")}
        core: Dict[str, Any] = {}
        sections: Dict[str, Dict[str, Any]] = {}

        def take(key: str, value: Any, where: str) -> None:
            if key in known:
                core[key] = value
            else:
                logger.debug("Ignoring unknown config field: %s%s", where, key)

        for key, value in data.items():
            if isinstance(value, dict):
                if key in _GROUPS:
                    for sub, v in value.items():
                        take(sub, v, key + ".")
                else:
                    sections[key] = dict(value)
            else:
                take(key, value, "")
        return cls(**core, _extensions=sections)

    @classmethod
    def _from_json(cls, path: str) -> "LoaderConfig":
        with open(path, "r") as f:
            return cls.from_dict(json.load(f))

    @classmethod
    def from_file(cls, path: str) -> "LoaderConfig":
        """Load a configuration file (JSON is the only format)."""
        return cls._from_json(path)

    def get_extension_config(self, name: str) -> Dict[str, Any]:
        """The settings section of loader ``name`` without the settings every loader shares."""
        return {k: v for k, v in self._extensions.get(name, {}).items()
                if k not in _SHARED_WITH_EVERY_LOADER}

    def create_parallel_kwargs(self) -> Dict[str, Any]:
        """Arguments for ``PipelineParallel``; without ``use_pipeline`` loading is strictly
        serial (``queue_size=-1``: one batch in device memory at a time)."""
        if not self.use_pipeline:
            return {"queue_size": -1}
        return {"max_concurrent_producers": self.max_concurrent_producers,
                "queue_size": self.queue_size, "use_tqdm_on_load": self.use_tqdm_on_load}


def load_config() -> LoaderConfig:
    env_path = os.environ.get(CONFIG_ENV_VAR)
    if env_path is not None:
        if not os.path.isfile(env_path):
            raise FileNotFoundError(f"Config file specified by {CONFIG_ENV_VAR} not found: {env_path}")
        return LoaderConfig.from_file(env_path)
    if os.path.isfile(DEFAULT_CONFIG_PATH):
        return LoaderConfig.from_file(DEFAULT_CONFIG_PATH)
    return LoaderConfig()
