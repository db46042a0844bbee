"""One registry from an architecture's name (config.json ``architectures[0]``) to the
class that reads its configuration and describes its model.

The reference only checks that the GGUF architecture string contains "qwen"
(src/model/qwen_config.cpp:36-40); here the lookup is exact and an unknown name
is an error that lists what is registered.
"""
from __future__ import annotations

from typing import Any, Dict

from ..errors import require

_ARCHITECTURES: Dict[str, Any] = {}


def register_architecture(name: str, config_class) -> None:
    """``config_class`` needs ``from_dict(dict)`` and, on its instances, ``to_model_spec()``
    and ``to_dict()``."""
    require(name not in _ARCHITECTURES, f"architecture '{name}' is already registered")
    _ARCHITECTURES[name] = config_class


def unregister_architecture(name: str) -> None:
    _ARCHITECTURES.pop(name, None)


def registered_architectures():
    return sorted(_ARCHITECTURES)


def config_class_for(name: str):
    require(name in _ARCHITECTURES,
            f"unknown architecture '{name}'; registered: {', '.join(registered_architectures()) or '(none)'}")
    return _ARCHITECTURES[name]


def config_from_dict(d: Dict[str, Any]):
    archs = d.get("architectures")
    require(isinstance(archs, list) and len(archs) >= 1 and isinstance(archs[0], str),
            "config.json: 'architectures' must be a non-empty list of names")
    return config_class_for(archs[0]).from_dict(d)


def config_from_model_dir(model_dir: str):
    from .qwen3 import read_config_json
    return config_from_dict(read_config_json(model_dir))
