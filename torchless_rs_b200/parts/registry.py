"""Registries of parts.  A part is looked up by the `kind` of its `PartSpec`;
anything may register a new kind, also code outside this package."""
from __future__ import annotations

from typing import Callable, Dict

MIXERS: Dict[str, type] = {}
FEED_FORWARDS: Dict[str, type] = {}
NORMS: Dict[str, type] = {}
POSITIONS: Dict[str, type] = {}
BLOCKS: Dict[str, type] = {}

_TABLES = {"mixer": MIXERS, "feed_forward": FEED_FORWARDS, "norm": NORMS,
           "position": POSITIONS, "block": BLOCKS}


def register(table: str, kind: str) -> Callable[[type], type]:
    def deco(cls: type) -> type:
        _TABLES[table][kind] = cls
        return cls
    return deco


def register_mixer(kind: str): return register("mixer", kind)
def register_feed_forward(kind: str): return register("feed_forward", kind)
def register_norm(kind: str): return register("norm", kind)
def register_position(kind: str): return register("position", kind)
def register_block(kind: str): return register("block", kind)


def lookup(table: str, kind: str) -> type:
    t = _TABLES[table]
    if kind not in t:
        raise KeyError(f"no {table} is registered under '{kind}'; known: {', '.join(sorted(t))}")
    return t[kind]
