"""Registries from a part's ``kind`` to the class that implements it.

Adding a norm, position encoding, mixer, feed-forward or block arrangement is one
``register_*`` call; a test can do it without touching this package.
"""
from __future__ import annotations

from typing import Callable, Dict

NORMS: Dict[str, type] = {}
POSITIONS: Dict[str, type] = {}
MIXERS: Dict[str, type] = {}
FEEDFORWARDS: Dict[str, type] = {}
BLOCKS: Dict[str, type] = {}
EMBEDDINGS: Dict[str, type] = {}
HEADS: Dict[str, type] = {}

_TABLES = {
    "norm": NORMS,
    "position": POSITIONS,
    "mixer": MIXERS,
    "feedforward": FEEDFORWARDS,
    "block": BLOCKS,
    "embedding": EMBEDDINGS,
    "head": HEADS,
}


class UnknownPart(KeyError):
    pass


def _register(table_name: str, kind: str) -> Callable[[type], type]:
    def wrap(cls: type) -> type:
        _TABLES[table_name][kind] = cls
        return cls

    return wrap


def register_norm(kind: str):
    return _register("norm", kind)


def register_position(kind: str):
    return _register("position", kind)


def register_mixer(kind: str):
    return _register("mixer", kind)


def register_feedforward(kind: str):
    return _register("feedforward", kind)


def register_block(kind: str):
    return _register("block", kind)


def register_embedding(kind: str):
    return _register("embedding", kind)


def register_head(kind: str):
    return _register("head", kind)


def lookup(table_name: str, kind: str) -> type:
    table = _TABLES[table_name]
    if kind not in table:
        raise UnknownPart(f"no {table_name} named `{kind}` is registered (known: {sorted(table)})")
    return table[kind]
