"""Token embedding and output projection
(crates/ai-engine-runtime/src/arch/embedding.rs:14-20,33-35; tied head:
crates/ai-engine-runtime/src/arch/model.rs:130-134)."""
from __future__ import annotations

import torch

from ..kernels import ops
from ..weights.loader import TensorSpec
from .base import Part


class TokenEmbedding(Part):
    """params: vocab_size, hidden_size, alternatives (names that may stand in).
    tensors: weight [vocab, hidden].  forward(ctx) -> float32 residual stream [T, hidden] of the
    step's tokens (`ctx.token_ids`; an embedding that depends on the place reads `ctx.positions`)."""

    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.vocab, self.hidden = int(spec.params["vocab_size"]), int(spec.params["hidden_size"])
        self.weight = None

    def tensor_specs(self):
        return [TensorSpec(self.spec.tensors["weight"], (self.vocab, self.hidden),
                           alternatives=tuple(self.spec.params.get("alternatives", ())))]

    def load(self, source):
        self.weight = source.get(self.spec.tensors["weight"])

    def forward(self, ctx):
        return ops.embed_gather(ctx.token_ids, self.weight, ctx.err)


class LMHead(Part):
    """params: vocab_size, hidden_size, alternatives, stored.  tensors: weight
    [vocab, hidden] (the embedding's name when tied).  forward(h [N, hidden]) ->
    float32 logits [N, vocab]."""

    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.vocab, self.hidden = int(spec.params["vocab_size"]), int(spec.params["hidden_size"])
        self.weight = None

    def tensor_specs(self):
        return [TensorSpec(self.spec.tensors["weight"], (self.vocab, self.hidden),
                           alternatives=tuple(self.spec.params.get("alternatives", ())),
                           stored=bool(self.spec.params.get("stored", True)))]

    def load(self, source):
        self.weight = source.get(self.spec.tensors["weight"])

    def weight_bytes(self):
        return self.weight.numel() * self.weight.element_size()

    def flops(self, tokens, keys=0.0):
        return 2.0 * tokens * self.vocab * self.hidden

    def forward(self, h, err=None):
        return ops.linear(h, self.weight, torch.float32, err)
