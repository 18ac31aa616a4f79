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
        self.block = 0

    def tensor_specs(self):
        t = self.spec.tensors
        return [TensorSpec(t["gate"], (self.inter, self.hidden)),
                TensorSpec(t["up"], (self.inter, self.hidden)),
                TensorSpec(t["down"], (self.hidden, self.inter))]

    def load(self, source):
        t = self.spec.tensors
        g, u = source.get(t["gate"]), source.get(t["up"])
        dt = torch.float32 if torch.float32 in (g.dtype, u.dtype) else g.dtype
        # bfloat16: 64 gate rows then their 64 up rows, tile by tile, so that a 128-row
        # weight tile of the tensor-core kernel holds both halves of 64 outputs
        self.block = ops.TC_SWIGLU_BLOCK if (dt == torch.bfloat16 and self.inter % ops.TC_SWIGLU_BLOCK == 0) else 0
        if self.block:
            b = self.block
            self.w_gu = torch.stack([g.view(-1, b, self.hidden), u.view(-1, b, self.hidden)], dim=1) \
                .reshape(2 * self.inter, self.hidden).contiguous()
        else:
            self.w_gu = torch.cat([g.to(dt), u.to(dt)], dim=0).contiguous()
        self.w_down = source.get(t["down"])

    def weight_bytes(self):
        return sum(w.numel() * w.element_size() for w in (self.w_gu, self.w_down))

    def flops(self, tokens, keys=0.0):
        return 2.0 * tokens * 3 * self.inter * self.hidden

    adds_in_place = True

    def forward(self, h, ctx, add_to=None):
        err = ctx.err if ctx is not None else None
        a = ops.linear_swiglu(h, self.w_gu, self.block, err)
        if add_to is not None and ops.linear_add(add_to, a, self.w_down):
            return None
        return ops.linear_parts(a, self.w_down, err)   # joins the residual in float32, inside the next norm
