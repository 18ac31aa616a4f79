"""The pre-norm residual block (crates/ai-engine-runtime/src/arch/block.rs:13-27):
x = x + mixer(norm(x)); x = x + ffn(norm(x)).

The residual stream stays float32.  A branch's output is not added by a kernel
of its own: it travels as `pending` into the next norm, which adds it in
float32, stores the sum and normalises it in one pass over the row.
"""
from __future__ import annotations

from .base import Block


class PreNormBlock(Block):
    roles = {"mixer_norm": "norm", "mixer": "mixer", "ffn_norm": "norm", "ffn": "feed_forward"}

    def __init__(self, spec, env, parts):
        super().__init__(spec, env)
        self.mixer_norm, self.mixer = parts["mixer_norm"], parts["mixer"]
        self.ffn_norm, self.ffn = parts["ffn_norm"], parts["ffn"]

    def forward(self, x, pending, ctx, caches):
        h = self.mixer_norm.forward(x, pending)
        if self.mixer.adds_in_place:      # a large step's output projection adds to the stream itself: a is None then
            a = self.mixer.forward(h, ctx, caches.get("mixer"), add_to=x)
        else:
            a = self.mixer.forward(h, ctx, caches.get("mixer"))
        h = self.ffn_norm.forward(x, a)
        if self.ffn.adds_in_place:
            return x, self.ffn.forward(h, ctx, add_to=x)
        return x, self.ffn.forward(h, ctx)
