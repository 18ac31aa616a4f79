"""A model put together from a `ModelSpec`: embedding, layers from parts, the
run order, final norm, head.  `forward(ctx, cache)` runs exactly the tokens of
the step context and returns float32 logits at the wanted rows
(crates/ai-engine-runtime/src/arch/model.rs:209-224 is the whole-sequence
version of the same chain).
"""
from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import torch

from ..weights.loader import TensorSpec, WeightSource
from .base import BuildEnv, KVRequest, Part, StateRequest
from .registry import lookup
from .spec import LayerSpec, ModelSpec, PartSpec

_ROLE_FAMILY = {"mixer": "mixer", "ffn": "feed_forward", "mixer_norm": "norm", "ffn_norm": "norm"}


def _family_of(role: str) -> str:
    if role in _ROLE_FAMILY:
        return _ROLE_FAMILY[role]
    if role.endswith("norm"):
        return "norm"
    raise KeyError(f"block role `{role}` has no part family")


class Layer:
    def __init__(self, spec: LayerSpec, env: BuildEnv):
        block_cls = lookup("block", spec.block)
        missing = [r for r in block_cls.roles if r not in spec.parts]
        if missing:
            raise ValueError(f"block `{spec.block}` needs parts for roles {missing}")
        self.parts: Dict[str, Part] = {
            role: lookup(_family_of(role), ps.kind)(ps, env) for role, ps in spec.parts.items()}
        self.block = block_cls(PartSpec(spec.block), env, self.parts)
        self.mixer = self.parts.get("mixer")


class Model:
    def __init__(self, spec: ModelSpec, dtype: torch.dtype, device="cuda"):
        self.spec = spec
        self.dtype = dtype
        self.device = torch.device(device)
        env = BuildEnv(spec.hidden_size, dtype, self.device)
        for name, ps in spec.position_encodings.items():
            env.position_encodings[name] = lookup("position_encoding", ps.kind)(ps, env)
        self.env = env
        self.embedding = lookup("embedding", spec.embedding.kind)(spec.embedding, env)
        self.layers: List[Layer] = [Layer(ls, env) for ls in spec.layers]
        self.final_norm = lookup("norm", spec.final_norm.kind)(spec.final_norm, env)
        self.lm_head = lookup("head", spec.lm_head.kind)(spec.lm_head, env)
        self.order = list(spec.order)
        for i, rs in enumerate(self.order):
            if not 0 <= rs.layer < len(self.layers):
                raise ValueError(f"run order entry {i} names layer {rs.layer}, which does not exist")
            if rs.cache_from is not None and not (0 <= rs.cache_from < i and
                                                  self.order[rs.cache_from].cache_from is None):
                raise ValueError(f"run order entry {i}: cache_from must name an earlier entry "
                                 f"that has a cache of its own")
        self.loaded = False

    # -- parts and tensors ---------------------------------------------------
    def all_parts(self) -> List[Part]:
        out: List[Part] = list(self.env.position_encodings.values()) + [self.embedding]
        for l in self.layers:
            out.extend(l.parts.values())
        out += [self.final_norm, self.lm_head]
        return out

    def tensor_specs(self) -> List[TensorSpec]:
        seen, out = set(), []
        for p in self.all_parts():
            for s in p.tensor_specs():
                if s.name not in seen:
                    seen.add(s.name)
                    out.append(s)
        return out

    def load(self, source: WeightSource) -> None:
        for p in self.all_parts():
            p.load(source)
        self.loaded = True

    # -- what the cache manager must provide ----------------------------------
    def cache_requests(self) -> List[Tuple[Optional[KVRequest], Optional[StateRequest], Optional[int]]]:
        """For each entry of the run order: (pages wanted, state wanted, cache_from)."""
        out = []
        for rs in self.order:
            m = self.layers[rs.layer].mixer
            kv = m.cache_request() if m is not None else None
            st = m.state_request() if m is not None else None
            out.append((kv if rs.cache_from is None else None, st, rs.cache_from))
        return out

    def has_host_parts(self) -> bool:
        """True when a part reads step data on the host inside forward (`host_side =
        True` on its class): such a model cannot be replayed from a captured graph."""
        return any(getattr(p, "host_side", False) for p in self.all_parts())

    def step_weight_bytes(self) -> int:
        """Bytes of weights one step reads: every part once per run, the head once."""
        total = self.lm_head.weight_bytes() + self.final_norm.weight_bytes()
        for rs in self.order:
            total += sum(p.weight_bytes() for p in self.layers[rs.layer].parts.values())
        return total

    # -- the forward pass of one step -----------------------------------------
    def forward(self, ctx, cache) -> torch.Tensor:
        x = self.embedding.forward(ctx.token_ids, ctx.err)
        pending = None
        for i, rs in enumerate(self.order):
            x, pending = self.layers[rs.layer].block.forward(x, pending, ctx, cache.layer_cache(i, ctx))
        if ctx.num_logit_rows == 0:
            return torch.empty((0, self.spec.vocab_size), dtype=torch.float32, device=self.device)
        h = self.final_norm.forward(x, pending, rows=ctx.logit_rows, write_back=False)
        return self.lm_head.forward(h, ctx.err)


def tensor_specs_of(spec: ModelSpec) -> List[TensorSpec]:
    """The tensors a model of this spec reads (no device needed)."""
    return Model(spec, torch.float32, device="cpu").tensor_specs()
