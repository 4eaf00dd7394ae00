"""One registry from an architecture's name to its typed configuration and model builder.

An architecture is two functions: ``config_from_dict(config.json, generation_config.json)``
returning its typed configuration, and ``build_spec(config)`` returning a ``ModelSpec``
(a list of blocks made of registered parts, and the order in which they run).  The
loader, cache manager, step function, scheduler, sampler and replay tool know nothing
else about a model.

Mirrors the role of lily/models/registry.py:13-47 (architectures[] name -> class;
an unknown name raises ``ValueError`` listing the supported ones, registry.py:40).
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Dict, List, Optional, Sequence


@dataclass
class Architecture:
    name: str
    config_from_dict: Callable[..., Any]     # (config.json dict, generation dict, architecture=name) -> config
    build_spec: Callable[[Any], Any]         # config -> ModelSpec


_ARCHITECTURES: Dict[str, Architecture] = {}
_BUILTINS_LOADED = False


def register_architecture(name: str, config_from_dict: Callable[..., Any],
                          build_spec: Callable[[Any], Any]) -> Architecture:
    arch = Architecture(name, config_from_dict, build_spec)
    _ARCHITECTURES[name] = arch
    return arch


def _load_builtins() -> None:
    global _BUILTINS_LOADED
    if not _BUILTINS_LOADED:
        _BUILTINS_LOADED = True
        import lily_b200.models  # noqa: F401  (registers the architectures this package ships)


def supported_architectures() -> List[str]:
    _load_builtins()
    return sorted(_ARCHITECTURES)


def resolve_architecture(architectures: Optional[Sequence[str]]) -> Architecture:
    _load_builtins()
    for name in architectures or []:
        if name in _ARCHITECTURES:
            return _ARCHITECTURES[name]
    raise ValueError(f"No registered model for architectures {list(architectures or [])}; "
                     f"have {sorted(_ARCHITECTURES)}")
