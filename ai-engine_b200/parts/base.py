"""Interfaces of the parts.

Every part is built from a `PartSpec` (sizes and constants as parameters) and a
`BuildEnv` (what the surrounding model provides: compute dtype, device, the
position encodings by name).  Building allocates nothing on the device;
`load(source)` fetches the part's tensors by name.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple

import torch

from ..weights.loader import TensorSpec, WeightSource
from .spec import PartSpec


@dataclass
class BuildEnv:
    hidden_size: int
    dtype: torch.dtype                      # compute dtype: torch.bfloat16 or torch.float32
    device: torch.device
    position_encodings: Dict[str, "Part"] = field(default_factory=dict)


@dataclass(frozen=True)
class KVRequest:
    """A mixer's need of a growing cache: keys and values of `kv_heads` x
    `head_dim` per token; `window` > 0: only the last `window` keys are read."""
    kv_heads: int
    head_dim: int
    window: int = 0


@dataclass(frozen=True)
class StateRequest:
    """A mixer's need of per-request state of fixed size, kept in a slot."""
    shape: Tuple[int, ...]
    dtype: torch.dtype = torch.float32


@dataclass
class LayerCache:
    """What a mixer gets of the cache for one run of its layer in one step."""
    k_pages: Optional[torch.Tensor] = None       # [num_pages, kv_heads, page, head_dim]
    v_pages: Optional[torch.Tensor] = None
    block_table: Optional[torch.Tensor] = None   # int32 [R, width], row r = request r of the batch
    page_size: int = 0
    writes: bool = True                          # False: the pages belong to another run; read only
    state: Optional[torch.Tensor] = None         # [max_seqs, *shape], row = the request's slot


class Part:
    def __init__(self, spec: PartSpec, env: BuildEnv):
        self.spec, self.env = spec, env

    def tensor_specs(self) -> List[TensorSpec]:
        return []

    def load(self, source: WeightSource) -> None:
        pass

    def weight_bytes(self) -> int:
        """Bytes of weights a step reads from this part (for the roofline)."""
        return 0


class Mixer(Part):
    """Mixes information across a request's tokens.  forward(h [T, hidden],
    ctx, cache) -> [T, hidden], float32 or the compute dtype (the next norm adds it to
    the float32 residual stream); float32 [parts, T, hidden] is taken too and summed there.  A part whose forward reads
    the step's host-side arrays (ctx.h_*) sets `host_side = True`; a model with such
    a part is never replayed from a captured CUDA graph."""

    host_side = False

    def cache_request(self) -> Optional[KVRequest]:
        return None

    def state_request(self) -> Optional[StateRequest]:
        return None

    def forward(self, h: torch.Tensor, ctx, cache: LayerCache) -> torch.Tensor:
        raise NotImplementedError


class FeedForward(Part):
    """Token-local: forward(h [T, hidden], ctx) -> [T, hidden], float32 or the compute dtype."""

    def forward(self, h: torch.Tensor, ctx) -> torch.Tensor:
        raise NotImplementedError


class Norm(Part):
    """forward(x, delta, rows, write_back): s = x (+ delta), stored into the
    float32 residual stream x when write_back; returns norm(s) in the compute
    dtype (only rows `rows` when given)."""

    def forward(self, x, delta=None, rows=None, write_back=True) -> torch.Tensor:
        raise NotImplementedError


class PositionEncoding(Part):
    """Owns the constants of a position encoding (for rotary: inv_freq)."""


class Block(Part):
    """An arrangement of parts.  forward(x, pending, ctx, cache) -> (x, pending):
    x is the float32 residual stream, `pending` a branch output not yet added
    (it is added inside the next norm)."""

    roles: Tuple[str, ...] = ()

    def forward(self, x, pending, ctx, cache: LayerCache):
        raise NotImplementedError
