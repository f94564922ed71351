"""Registries of part kinds.  A configuration names parts by kind, layer by layer;
the model builder looks the kind up here and calls it with the parameters.

    register_mixer("my_mixer", MyMixer)         # MyMixer(**params)

Nothing else has to change for a new kind to be built, loaded and stepped.
"""
from __future__ import annotations

from typing import Callable, Dict

from ..errors import ErrorCode, PhotonError

NORMS: Dict[str, Callable] = {}
MIXERS: Dict[str, Callable] = {}
FEED_FORWARDS: Dict[str, Callable] = {}
POSITION_ENCODINGS: Dict[str, Callable] = {}
BLOCKS: Dict[str, Callable] = {}

_TABLES = {"norm": NORMS, "mixer": MIXERS, "feed_forward": FEED_FORWARDS,
           "position_encoding": POSITION_ENCODINGS, "block": BLOCKS}


def _register(table_name: str, kind: str, factory: Callable, replace: bool) -> None:
    table = _TABLES[table_name]
    if kind in table and not replace:
        raise PhotonError(ErrorCode.INVALID_ARGUMENT, f"{table_name} kind {kind!r} is already registered")
    table[kind] = factory


def register_norm(kind, factory, replace=False): _register("norm", kind, factory, replace)
def register_mixer(kind, factory, replace=False): _register("mixer", kind, factory, replace)
def register_feed_forward(kind, factory, replace=False): _register("feed_forward", kind, factory, replace)
def register_position_encoding(kind, factory, replace=False): _register("position_encoding", kind, factory, replace)
def register_block(kind, factory, replace=False): _register("block", kind, factory, replace)


def create_part(table_name: str, kind: str, params: dict):
    _ensure_builtin()
    table = _TABLES[table_name]
    if kind not in table:
        known = ", ".join(sorted(table)) or "none"
        raise PhotonError(ErrorCode.UNSUPPORTED_MODEL,
                          f"{table_name} kind {kind!r} is not registered (known: {known})")
    return table[kind](**params)


def _ensure_builtin() -> None:
    from . import attention, block, mlp, norm, rope  # noqa: F401  (each registers itself)
