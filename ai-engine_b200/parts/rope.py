"""Rotary position encoding: the frequencies.

Default (crates/ai-engine-runtime/src/arch/rope.rs:34-36): inv_freq[i] =
1 / theta^(2i/d) in float32.  The reference precomputes cos/sin tables up to
max_position_embeddings; here only inv_freq is kept and kernels compute
cos/sin(float(pos) * inv_freq[i]) in float32, so no table bounds the context.

`llama3` scaling is not in the reference (it reads no rope_scaling); it follows
the rule the config keys name: with wavelength = 2*pi / inv_freq, frequencies
whose wavelength is below original/high_freq_factor are kept, above
original/low_freq_factor are divided by `factor`, and between the two are
blended linearly in original/wavelength.
"""
from __future__ import annotations

import math

import numpy as np
import torch

from .base import PositionEncoding


def rotary_inv_freq(rot_dim: int, theta: float, scaling=None) -> np.ndarray:
    i = np.arange(rot_dim // 2, dtype=np.float32)
    base = (np.float32(1.0) / np.power(np.float32(theta), (np.float32(2.0) * i) / np.float32(rot_dim)))
    base = base.astype(np.float32)
    if not scaling:
        return base
    kind = scaling.get("rope_type", scaling.get("type"))
    if kind != "llama3":
        raise ValueError(f"rotary scaling `{kind}` is not supported (supported: llama3)")
    factor = float(scaling["factor"])
    low, high = float(scaling["low_freq_factor"]), float(scaling["high_freq_factor"])
    original = float(scaling["original_max_position_embeddings"])
    f = base.astype(np.float64)
    wavelength = 2.0 * math.pi / f
    smooth = (original / wavelength - low) / (high - low)
    blended = (1.0 - smooth) * f / factor + smooth * f
    out = np.where(wavelength < original / high, f,
                   np.where(wavelength > original / low, f / factor, blended))
    return out.astype(np.float32)


class RotaryEncoding(PositionEncoding):
    """params: rot_dim (elements of each head that are rotated; the full head for
    Llama), theta, scaling (None or the llama3 dict).  Holds inv_freq
    [rot_dim / 2] float32 on the device."""

    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.rot_dim = int(spec.params["rot_dim"])
        if self.rot_dim % 2:
            raise ValueError(f"rotary encoding needs an even rot_dim, got {self.rot_dim}")
        self.inv_freq_host = rotary_inv_freq(self.rot_dim, float(spec.params["theta"]),
                                             spec.params.get("scaling"))
        self.inv_freq = None

    def load(self, source):
        self.inv_freq = torch.from_numpy(self.inv_freq_host.copy()).to(self.env.device)

    def rotation(self):
        return self.inv_freq, self.rot_dim
