"""One registry from an architecture's name (``architectures[0]`` of config.json) to
its configuration class and to the function that turns a configuration into a
``ModelSpec`` (the list of layers, their parts and the order they run in).

The reference has one hard-wired model class (include/photon/arch/llama_model.hpp:61)
and no registry; adding an architecture here is one ``register_architecture`` call.
"""
from __future__ import annotations

import dataclasses
from typing import Any, Callable, Dict

from ..errors import ErrorCode, PhotonError
from .model_config import read_config_json


@dataclasses.dataclass(frozen=True)
class Architecture:
    name: str
    config_class: Any                       # has from_dict(dict) and to_dict()
    build_spec: Callable[[Any], Any]        # config -> models.spec.ModelSpec


_ARCHITECTURES: Dict[str, Architecture] = {}


def register_architecture(name: str, config_class: Any, build_spec: Callable[[Any], Any],
                          replace: bool = False) -> None:
    if name in _ARCHITECTURES and not replace:
        raise PhotonError(ErrorCode.INVALID_ARGUMENT, f"architecture {name!r} is already registered")
    _ARCHITECTURES[name] = Architecture(name, config_class, build_spec)


def get_architecture(name: str) -> Architecture:
    _ensure_builtin()
    if name not in _ARCHITECTURES:
        known = ", ".join(sorted(_ARCHITECTURES)) or "none"
        raise PhotonError(ErrorCode.UNSUPPORTED_MODEL,
                          f"architecture {name!r} is not registered (known: {known})")
    return _ARCHITECTURES[name]


def registered_architectures():
    _ensure_builtin()
    return sorted(_ARCHITECTURES)


def load_config(path: str):
    """Read ``config.json`` and return ``(architecture, typed config)``."""
    d = read_config_json(path)
    archs = d.get("architectures")
    if not isinstance(archs, list) or not archs:
        raise PhotonError(ErrorCode.INVALID_CONFIG, "config.json: key 'architectures' must be a non-empty list")
    arch = get_architecture(archs[0])
    return arch, arch.config_class.from_dict(d)


def _ensure_builtin() -> None:
    # importing the model module registers it
    from ..models import llama  # noqa: F401
