"""String-keyed registry of copier factories (as upstream ``copier/registry.py``).

A factory is called once per loader with the target device and the loader's keyword
arguments; it returns the function that builds one copier per file.
"""

from __future__ import annotations

from typing import Any, Callable, Dict

CopierType = str
CopierConstructFunc = Callable[[Any, Any, Any], Any]
CopierConstructorFactory = Callable[..., CopierConstructFunc]

_factories: Dict[CopierType, CopierConstructorFactory] = {}


def register_copier_constructor(copier_type: CopierType):
    def remember(factory: CopierConstructorFactory) -> CopierConstructorFactory:
        _factories[copier_type] = factory
        return factory

    return remember


def create_copier_constructor(copier_type: CopierType, device, **kwargs) -> CopierConstructFunc:
    try:
        factory = _factories[copier_type]
    except KeyError:
        raise KeyError(
            f"Copier type '{copier_type}' is not registered. Available types: {list(_factories.keys())}"
        ) from None
    return factory(device, **kwargs)
