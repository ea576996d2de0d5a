"""``AutoLoader``: the pipelined iterator configured from a file instead of arguments
(upstream ``fastsafetensors/auto_loader.py``).  Only the ``"base"`` loader exists here."""

from __future__ import annotations

from typing import Any, Dict, Generator, List, Optional, Tuple, Type

from .common import init_logger
from .config import LoaderConfig, load_config
from .loader import BaseSafeTensorsFileLoader, SafeTensorsFileLoader
from .parallel_loader import PipelineParallel

logger = init_logger(__name__)

# loader name -> name of a class in this module (looked up at call time, so tests can patch it)
_LOADER_REGISTRY: Dict[str, str] = {"base": "SafeTensorsFileLoader"}


def _resolve_loader_class(loader_name: str) -> Type[BaseSafeTensorsFileLoader]:
    attr = _LOADER_REGISTRY.get(loader_name)
    if attr is None:
        raise ValueError(f"Unknown loader type: {loader_name!r}. Available: {list(_LOADER_REGISTRY)}")
    cls = globals().get(attr)
    if cls is None:
        raise ValueError(f"Loader class '{attr}' for loader type {loader_name!r} is not imported in this module.")
    return cls


class AutoLoader:
    """``for key, tensor in AutoLoader(pg, files, device="cuda:0").iterate_weights(): ...``"""

    def __init__(self, pg: Optional[Any], hf_weights_files: List[str], device: Any = "cpu"):
        cfg = self._config = load_config()
        loader_cls = _resolve_loader_class(cfg.loader)
        ext = loader_cls.process_extension_config(cfg.get_extension_config(cfg.loader),
                                                  hf_weights_files=hf_weights_files)
        self._loader = loader_cls(pg, device=device, framework=cfg.framework, debug_log=cfg.debug_log,
                                  set_numa=cfg.set_numa, disable_cache=cfg.disable_cache, **ext)
        self._pipeline = PipelineParallel(pg=pg, loader=self._loader, hf_weights_files=hf_weights_files,
                                          **cfg.create_parallel_kwargs())
        logger.info("AutoLoader initialized: loader=%s, device=%s, files=%d, %s", cfg.loader, device,
                    len(hf_weights_files), ", ".join(f"{k}={v}" for k, v in ext.items()))

    @property
    def config(self) -> LoaderConfig:
        return self._config

    def iterate_weights(self) -> Generator[Tuple[str, Any], None, None]:
        return self._pipeline.iterate_weights()

    def close(self) -> None:
        self._pipeline.close()   # closes the loader too
