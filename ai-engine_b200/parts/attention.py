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

from ..kernels import ops
from ..weights.loader import TensorSpec
from .base import KVRequest, Mixer


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
        if self.rope is not None and self.rope.rot_dim > self.d:
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

    def cache_request(self):
        return KVRequest(self.K, self.d, self.window)

    def forward(self, h, ctx, cache):
        inv_freq = self.rope.inv_freq if self.rope is not None else self._no_rope
        # a small bfloat16 step: product, rotation and cache write in one kernel
        q = ops.linear_rope_kv(h, self.w_qkv, cache.k_pages, cache.v_pages, ctx.positions, ctx.token_req,
                               cache.block_table, inv_freq, self.H, self.K, self.d, ctx.err,
                               write=cache.writes)
        if q is None:
            qkv = ops.linear_parts(h, self.w_qkv, ctx.err, self.env.dtype)
            q = ops.rope_kv_write(qkv, cache.k_pages, cache.v_pages, ctx.positions, ctx.token_req,
                                  cache.block_table, inv_freq, self.H, self.K, self.d, ctx.err,
                                  write=cache.writes)
        a = ops.paged_attention(q, cache.k_pages, cache.v_pages, ctx, cache.block_table,
                                self.scale, self.window)
        return ops.linear_parts(a.view(a.shape[0], self.H * self.d), self.w_o, ctx.err)
