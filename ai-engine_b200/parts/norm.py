"""RMSNorm (crates/ai-engine-runtime/src/arch/rmsnorm.rs:29-42)."""
from __future__ import annotations

from ..kernels import ops
from ..weights.loader import TensorSpec
from .base import Norm


class RMSNorm(Norm):
    """params: size, eps.  tensors: weight [size].  y = (x / sqrt(mean(x^2) + eps)) * w,
    statistics in float32; the add of a pending branch is fused in."""

    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.size = int(spec.params["size"])
        self.eps = float(spec.params["eps"])
        self.weight = None

    def tensor_specs(self):
        return [TensorSpec(self.spec.tensors["weight"], (self.size,), init="ones")]

    def load(self, source):
        self.weight = source.get(self.spec.tensors["weight"])

    def weight_bytes(self):
        return self.weight.numel() * self.weight.element_size()

    def forward(self, x, delta=None, rows=None, write_back=True):
        return ops.add_rmsnorm(x, delta, self.weight, self.eps, self.env.dtype, rows=rows,
                               write_back=write_back)
