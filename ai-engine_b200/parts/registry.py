"""Registries of part kinds.  A part is chosen by `PartSpec.kind`, layer by layer."""
from __future__ import annotations

from typing import Dict

MIXERS: Dict[str, type] = {}
FEED_FORWARDS: Dict[str, type] = {}
NORMS: Dict[str, type] = {}
POSITION_ENCODINGS: Dict[str, type] = {}
BLOCKS: Dict[str, type] = {}
EMBEDDINGS: Dict[str, type] = {}
HEADS: Dict[str, type] = {}

_ALL = {"mixer": MIXERS, "feed_forward": FEED_FORWARDS, "norm": NORMS,
        "position_encoding": POSITION_ENCODINGS, "block": BLOCKS, "embedding": EMBEDDINGS,
        "head": HEADS}


def register(family: str, kind: str, cls: type) -> None:
    """Add a part class.  family: mixer | feed_forward | norm | position_encoding |
    block | embedding | head."""
    _ALL[family][kind] = cls


def register_mixer(kind: str, cls: type) -> None:
    register("mixer", kind, cls)


def register_feed_forward(kind: str, cls: type) -> None:
    register("feed_forward", kind, cls)


def register_norm(kind: str, cls: type) -> None:
    register("norm", kind, cls)


def register_position_encoding(kind: str, cls: type) -> None:
    register("position_encoding", kind, cls)


def register_block(kind: str, cls: type) -> None:
    register("block", kind, cls)


def lookup(family: str, kind: str) -> type:
    table = _ALL[family]
    if kind not in table:
        raise KeyError(f"no {family} part of kind `{kind}` is registered "
                       f"(registered: {', '.join(sorted(table)) or 'none'})")
    return table[kind]
