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
from .base import BuildEnv, CacheNeed, Part, StepPlanner
from .registry import lookup
from .spec import LayerSpec, ModelSpec, PartSpec


class Layer:
    """The parts of one layer, built by the families that its block names for its roles."""

    def __init__(self, spec: LayerSpec, env: BuildEnv):
        block_cls = lookup("block", spec.block)
        roles = dict(block_cls.roles)
        missing = [r for r in roles if r not in spec.parts]
        unknown = [r for r in spec.parts if r not in roles]
        if missing or unknown:
            raise ValueError(f"block `{spec.block}` has the roles {sorted(roles)}: "
                             f"missing parts for {missing}, no role for {unknown}")
        self.parts: Dict[str, Part] = {
            role: lookup(roles[role], spec.parts[role].kind)(spec.parts[role], env) for role in roles}
        self.block = block_cls(PartSpec(spec.block), env, self.parts)

    def cache_needs(self):
        """(role, pages wanted, state wanted) of every part that asks for either."""
        out = []
        for role, part in self.parts.items():
            kv, st = part.cache_request(), part.state_request()
            if kv is not None or st is not None:
                out.append((role, kv, st))
        return out


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
        wanted: Dict[str, int] = {}
        for p in self.all_parts():
            for s in p.tensor_specs():
                wanted[s.name] = wanted.get(s.name, 0) + 1
        source.keep_only([n for n, c in wanted.items() if c > 1])
        for p in self.all_parts():
            p.load(source)
        self.loaded = True

    # -- what the cache manager must provide ----------------------------------
    def cache_requests(self) -> List[CacheNeed]:
        """What the parts of every run-order entry ask of the cache manager.  An entry that reads
        another entry's cache gets that entry's pages, role by role, and none of its own."""
        out = []
        for i, rs in enumerate(self.order):
            for role, kv, st in self.layers[rs.layer].cache_needs():
                if rs.cache_from is not None and kv is not None:
                    out.append(CacheNeed(i, role, None, st, rs.cache_from))
                else:
                    out.append(CacheNeed(i, role, kv, st, None))
        return out

    def step_planners(self) -> List[StepPlanner]:
        """The planners whose lists the parts read in forward, each once."""
        out: List[StepPlanner] = []
        for p in self.all_parts():
            pl = p.step_planner()
            if pl is not None and all(pl is not q for q in out):
                out.append(pl)
        return out

    def keeps_state(self) -> bool:
        return any(n.state is not None for n in self.cache_requests())

    def pads_decode_rows(self) -> bool:
        """Whether decode steps may be rounded up by repeating a row: every part that keeps state
        skips rows with `ctx.live == 0`."""
        return all(getattr(p, "skips_padded_rows", False) or p.state_request() is None
                   for l in self.layers for p in l.parts.values())

    def has_host_parts(self) -> bool:
        """True when a part reads step data on the host inside forward (`host_side =
        True` on its class): such a model cannot be replayed from a captured graph."""
        return any(getattr(p, "host_side", False) for p in self.all_parts())

    def step_flops(self, tokens: int, keys: float = 0.0, logit_rows: int = 1) -> float:
        """Floating-point operations of one step of `tokens` tokens that read `keys` cached positions
        each on average, with logits at `logit_rows` rows: every part once per run, the head once."""
        total = self.lm_head.flops(logit_rows) + self.final_norm.flops(logit_rows)
        for rs in self.order:
            total += sum(p.flops(tokens, keys) for p in self.layers[rs.layer].parts.values())
        return total

    def step_weight_bytes(self) -> int:
        """Bytes of weights one step reads: every part once per run, the head once."""
        total = self.lm_head.weight_bytes() + self.final_norm.weight_bytes()
        for rs in self.order:
            total += sum(p.weight_bytes() for p in self.layers[rs.layer].parts.values())
        return total

    # -- the forward pass of one step -----------------------------------------
    def forward(self, ctx, cache) -> torch.Tensor:
        x = self.embedding.forward(ctx)
        for pe in self.env.position_encodings.values():
            pe.add_to(x, ctx)
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
