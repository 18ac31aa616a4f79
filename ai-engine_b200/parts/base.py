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


@dataclass(frozen=True)
class CacheNeed:
    """What one part of one run-order entry asks of the cache manager: pages (`kv`), a
    slot-indexed state tensor (`state`), or another run's pages read without writing
    (`cache_from`: the index of that run-order entry; `kv` is None then)."""
    run: int
    role: str
    kv: Optional[KVRequest] = None
    state: Optional[StateRequest] = None
    cache_from: Optional[int] = None


class StepPlanner:
    """Derived index lists that a kind of part wants for every step (for attention: which tokens are lone
    decoded tokens, which tiles the prompt portions fall into).  `plan(ctx)` is called on the host with the
    step's generic arrays (`ctx.h_q_start / h_q_len / h_ctx_len / h_slots`, `T`, `R`, `bt_width`,
    `page_size`, `bucketed`) and returns (int32 arrays by name, host scalars by name).  The arrays travel
    in the step's one packed buffer; a part reads them back with `ctx.plan(planner)`.  Parts that return
    the same planner object share one plan.  For steps that may be replayed from a captured graph
    (`ctx.bucketed`), lengths of the arrays and the scalars must depend on the layout only (R, T, bt_width)."""

    key: str = ""

    def plan(self, ctx):
        raise NotImplementedError


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

    def flops(self, tokens: int, keys: float = 0.0) -> float:
        """Floating-point operations of one forward over `tokens` tokens that each read `keys` cached
        positions on average (for the roofline; 2 per multiply-add)."""
        return 0.0

    def cache_request(self) -> Optional[KVRequest]:
        """Pages this part wants (any part of a block may ask, not only the one in the role `mixer`)."""
        return None

    def state_request(self) -> Optional[StateRequest]:
        """Per-request state of fixed size this part wants."""
        return None

    def step_planner(self) -> Optional[StepPlanner]:
        """The planner whose lists this part reads in forward (None: the generic arrays suffice)."""
        return None


class Mixer(Part):
    """Mixes information across a request's tokens.  forward(h [T, hidden],
    ctx, cache) -> [T, hidden], float32 or the compute dtype (the next norm adds it to
    the float32 residual stream); float32 [parts, T, hidden] is taken too and summed there.  A part whose forward reads
    the step's host-side arrays (ctx.h_*) sets `host_side = True`; a model with such
    a part is never replayed from a captured CUDA graph.

    Decode steps that are replayed from a graph are rounded up to a multiple of 8 rows by repeating the
    first entry; `ctx.live[r]` is 0 for such a row.  Attention may ignore it (the row writes the same key
    and value again).  A part that keeps state must not update it for those rows; it says that it checks by
    `skips_padded_rows = True`, otherwise its model's steps are never rounded up."""

    host_side = False
    skips_padded_rows = False
    # True: forward takes `add_to=stream` (the float32 residual stream) and may add its output there itself,
    # returning None instead of the output (a block then hands no pending branch to the next norm)
    adds_in_place = False

    def forward(self, h: torch.Tensor, ctx, cache: LayerCache) -> torch.Tensor:
        raise NotImplementedError


class FeedForward(Part):
    """Token-local: forward(h [T, hidden], ctx) -> [T, hidden], float32 or the compute dtype."""

    adds_in_place = False      # as for a Mixer

    def forward(self, h: torch.Tensor, ctx) -> torch.Tensor:
        raise NotImplementedError


class Norm(Part):
    """forward(x, delta, rows, write_back): s = x (+ delta), stored into the
    float32 residual stream x when write_back; returns norm(s) in the compute
    dtype (only rows `rows` when given)."""

    def forward(self, x, delta=None, rows=None, write_back=True) -> torch.Tensor:
        raise NotImplementedError


class PositionEncoding(Part):
    """Owns the constants of a position encoding and says how it acts.  Two ways, both optional:

    * `rotation()` -> (inv_freq float32 [rot_dim / 2] on the device, rot_dim): a mixer rotates the first
      `rot_dim` elements of its queries and keys by position * inv_freq (split halves).  Another base,
      scaling rule or a partial rotation is another vector or width.  None: no rotation.
    * `add_to(x, ctx)`: adds the encoding of `ctx.positions` into the float32 residual stream `x`
      [T, hidden] in place, right after the embedding (learned or fixed absolute encodings).
    """

    def rotation(self):
        return None

    def add_to(self, x, ctx) -> None:
        return None


class Block(Part):
    """An arrangement of parts.  `roles` maps each role of the arrangement to the family its part is
    looked up in (mixer | feed_forward | norm).  forward(x, pending, ctx, caches) -> (x, pending):
    x is the float32 residual stream, `pending` a branch output not yet added (it is added inside the
    next norm); `caches[role]` is the LayerCache of the part in that role (only roles whose part asked
    for pages or state have one)."""

    roles: Dict[str, str] = {}

    def forward(self, x, pending, ctx, caches: Dict[str, LayerCache]):
        raise NotImplementedError
