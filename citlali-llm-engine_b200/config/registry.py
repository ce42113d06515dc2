"""One registry from an architecture's name (config.json ``architectures[0]``, or ``architecture``) to the
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


def architecture_name(d: Dict[str, Any]) -> str:
    """``architectures[0]``, or, in a config.json that has no such list, the string ``architecture``."""
    archs = d.get("architectures")
    if archs is None and isinstance(d.get("architecture"), str):
        return d["architecture"]
    require(isinstance(archs, list) and len(archs) >= 1 and isinstance(archs[0], str),
            "config.json: 'architectures' must be a non-empty list of names (or 'architecture' one name)")
    return archs[0]


def config_from_dict(d: Dict[str, Any]):
    return config_class_for(architecture_name(d)).from_dict(d)


def config_from_model_dir(model_dir: str):
    """The configuration of a model folder.  A class whose design leaves some sizes to the shapes of the checkpoint's
    tensors offers ``with_tensor_shapes({name: shape})``; it is then given the shapes the folder's weight files declare
    (their headers are read, no values)."""
    from .qwen3 import read_config_json
    config = config_from_dict(read_config_json(model_dir))
    if callable(getattr(config, "with_tensor_shapes", None)):
        from ..weights.loader import WeightLoader
        loader = WeightLoader(model_dir)
        try:
            config = config.with_tensor_shapes({n: tuple(loader.stored_shape(n)) for n in loader.names()})
        finally:
            loader.close()
    return config
