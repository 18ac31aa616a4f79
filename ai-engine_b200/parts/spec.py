"""A model as data: which parts each layer is made of, with their sizes and
constants, which tensors they read, and in which order layers run.

An architecture's `build_spec(config)` returns a `ModelSpec`; nothing below it
knows which model it is in.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple


@dataclass
class PartSpec:
    """One part: its registered kind, its sizes and constants, and the names of
    the tensors it reads (role -> tensor name)."""
    kind: str
    params: Dict[str, object] = field(default_factory=dict)
    tensors: Dict[str, str] = field(default_factory=dict)


@dataclass
class LayerSpec:
    """One layer: the arrangement (`block`, a registered block kind) and the parts
    that fill its roles (for the pre-norm block: mixer_norm, mixer, ffn_norm, ffn)."""
    block: str
    parts: Dict[str, PartSpec]


@dataclass
class RunStep:
    """One entry of the run order.  `layer` indexes `ModelSpec.layers` (a layer may
    be named by several entries).  `cache_from`: the index of an earlier entry
    whose cache this one reads without writing; None: a cache of its own."""
    layer: int
    cache_from: Optional[int] = None


@dataclass
class ModelSpec:
    hidden_size: int
    vocab_size: int
    max_position: int
    embedding: PartSpec
    layers: List[LayerSpec]
    order: List[RunStep]
    final_norm: PartSpec
    lm_head: PartSpec
    position_encodings: Dict[str, PartSpec] = field(default_factory=dict)
    eos_token_ids: Tuple[int, ...] = ()
    ignored_tensors: Tuple[str, ...] = ()     # name endings of stored tensors that are no parameters
