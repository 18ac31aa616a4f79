"""SwiGLU feed-forward (crates/ai-engine-runtime/src/arch/ffn.rs:50-54):
down(silu(gate(x)) * up(x)), no bias, silu(z) = z * sigmoid(z) in float32."""
from __future__ import annotations

import torch

from ..kernels import ops
from ..weights.loader import TensorSpec
from .base import FeedForward


class SwiGLU(FeedForward):
    """params: hidden_size, intermediate_size.  tensors: gate, up [F, hidden],
    down [hidden, F].  gate and up are fused into one [2F, hidden] weight at load."""

    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.hidden = int(spec.params["hidden_size"])
        self.inter = int(spec.params["intermediate_size"])
        self.w_gu = self.w_down = None

    def tensor_specs(self):
        t = self.spec.tensors
        return [TensorSpec(t["gate"], (self.inter, self.hidden)),
                TensorSpec(t["up"], (self.inter, self.hidden)),
                TensorSpec(t["down"], (self.hidden, self.inter))]

    def load(self, source):
        t = self.spec.tensors
        g, u = source.get(t["gate"]), source.get(t["up"])
        dt = torch.float32 if torch.float32 in (g.dtype, u.dtype) else g.dtype
        self.w_gu = torch.cat([g.to(dt), u.to(dt)], dim=0).contiguous()
        self.w_down = source.get(t["down"])

    def weight_bytes(self):
        return sum(w.numel() * w.element_size() for w in (self.w_gu, self.w_down))

    def forward(self, h, ctx):
        a = ops.linear_swiglu(h, self.w_gu)
        return ops.linear(a, self.w_down, torch.float32)     # the branch joins the residual in float32
