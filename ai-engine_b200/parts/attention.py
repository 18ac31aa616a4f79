"""Grouped-query attention over the paged cache.

Formula (crates/ai-engine-runtime/src/arch/attention.rs:114-166): q, k, v
projections without bias; rotary encoding of q and k at each token's absolute
position; k, v appended to the cache before it is read; query head h reads kv
head h / (H/K) (:177-196); scores = (q.k) * scale with scale = 1/sqrt(d) applied
after the dot product (:53,153-154); key j visible to a query at p iff j <= p
(:203-224); softmax in float32; context . Wo.
"""
from __future__ import annotations

import math

import torch

import numpy as np

from ..kernels import ops
from ..weights.loader import TensorSpec
from .base import KVRequest, Mixer, StepPlanner


class AttentionWork(StepPlanner):
    """The work lists of the attention kernels, derived from a step's generic arrays: `decode_tokens`
    (rows of requests that bring one token, for the split-KV kernel), `other_tokens` (rows of all others),
    `prefill_tiles` [n, 2] = (request row, offset of a tile of `ops.PREFILL_TILE` tokens among the tokens it
    brings), `prefill_pairs` [m, 2] = the same in units of two tiles (for the kernel whose CTAs take two),
    `n_decode`, and `max_decode_len`.  The lone-token rows are listed longest context first: the
    decode kernel's CTAs start in that order, so when there are more of them than fit the machine at once the
    long requests do not start last (the most keys a lone token reads: of the layout's widest
    possible request when the step may be replayed from a graph)."""

    key = "attention"

    def plan(self, ctx):
        # the lists are made by the host runtime (csrc/host/step_pack.hpp:attention_lists)
        from ..cache.manager import host as host_runtime

        dec, other, tiles, pairs, n_decode, max_decode_len = host_runtime().attention_lists(
            ctx.h_q_start, ctx.h_q_len, ctx.h_ctx_len, ops.PREFILL_TILE)
        if ctx.bucketed and n_decode:
            max_decode_len = ctx.bt_width * ctx.page_size      # a property of the layout, not of the step
        return (dict(decode_tokens=dec, other_tokens=other, prefill_tiles=tiles, prefill_pairs=pairs),
                dict(n_decode=n_decode, max_decode_len=max_decode_len))


ATTENTION_WORK = AttentionWork()


class GQAAttention(Mixer):
    """params: hidden_size, num_heads, num_kv_heads, head_dim, window (0 = all
    keys), scale (None = 1/sqrt(head_dim)), position_encoding (name of a rotary
    encoding of the model, or None).  tensors: q, k, v [heads*d, hidden], o
    [hidden, H*d].  q, k, v are fused into one [(H + 2K) * d, hidden] weight at load."""

    def __init__(self, spec, env):
        super().__init__(spec, env)
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.H, self.K, self.d = int(p["num_heads"]), int(p["num_kv_heads"]), int(p["head_dim"])
        if self.H % self.K:
            raise ValueError(f"attention: {self.H} heads are not a multiple of {self.K} kv heads")
        if self.d % 16 or self.d > 256:
            raise ValueError(f"attention: head_dim {self.d} must be a multiple of 16, at most 256")
        self.window = int(p.get("window") or 0)
        self.scale = float(p["scale"]) if p.get("scale") is not None else 1.0 / math.sqrt(self.d)
        pe = p.get("position_encoding")
        self.rope = env.position_encodings[pe] if pe else None
        rot = self.rope.rotation() if self.rope is not None else None
        if rot is not None and rot[1] > self.d:
            raise ValueError("attention: rotary width exceeds head_dim")
        self.w_qkv = self.w_o = None
        self._no_rope = None

    def tensor_specs(self):
        t = self.spec.tensors
        return [TensorSpec(t["q"], (self.H * self.d, self.hidden)),
                TensorSpec(t["k"], (self.K * self.d, self.hidden)),
                TensorSpec(t["v"], (self.K * self.d, self.hidden)),
                TensorSpec(t["o"], (self.hidden, self.H * self.d))]

    def load(self, source):
        t = self.spec.tensors
        q, k, v = source.get(t["q"]), source.get(t["k"]), source.get(t["v"])
        dt = torch.float32 if torch.float32 in (q.dtype, k.dtype, v.dtype) else q.dtype
        self.w_qkv = torch.cat([q.to(dt), k.to(dt), v.to(dt)], dim=0).contiguous()
        self.w_o = source.get(t["o"])
        self._no_rope = torch.zeros(0, dtype=torch.float32, device=self.env.device)

    def weight_bytes(self):
        return sum(w.numel() * w.element_size() for w in (self.w_qkv, self.w_o))

    def flops(self, tokens, keys=0.0):
        proj = 2.0 * tokens * self.hidden * (2 * self.H + 2 * self.K) * self.d
        return proj + 4.0 * tokens * keys * self.H * self.d         # q.k and p.v

    def cache_request(self):
        return KVRequest(self.K, self.d, self.window)

    def step_planner(self):
        return ATTENTION_WORK

    adds_in_place = True

    def forward(self, h, ctx, cache, add_to=None):
        rot = self.rope.rotation() if self.rope is not None else None
        inv_freq = rot[0] if rot is not None else self._no_rope
        # a small bfloat16 step: product, rotation and cache write in one kernel
        q = ops.linear_rope_kv(h, self.w_qkv, cache.k_pages, cache.v_pages, ctx.positions, ctx.token_req,
                               cache.block_table, inv_freq, self.H, self.K, self.d, ctx.err,
                               write=cache.writes)
        if q is None:
            # the projection reaches the rotation in float32 whatever the step's size (unjoined parts of a
            # small step, the library product's float32 output of a large one): q and k are rounded to
            # the cache's dtype once, after the rotation, so a key's bits do not depend on how its prompt was cut
            qkv = ops.linear_parts(h, self.w_qkv, ctx.err, torch.float32)
            q = ops.rope_kv_write(qkv, cache.k_pages, cache.v_pages, ctx.positions, ctx.token_req,
                                  cache.block_table, inv_freq, self.H, self.K, self.d, ctx.err,
                                  write=cache.writes)
        a = ops.paged_attention(q, cache.k_pages, cache.v_pages, ctx, ctx.plan(ATTENTION_WORK),
                                cache.block_table, self.scale, self.window)
        a = a.view(a.shape[0], self.H * self.d)
        if add_to is not None and ops.linear_add(add_to, a, self.w_o):
            return None
        return ops.linear_parts(a, self.w_o, ctx.err)
