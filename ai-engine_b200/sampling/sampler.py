"""Runs the sampling kernel over the rows of a step's logits."""
from __future__ import annotations

from ctypes import c_int
from typing import Sequence

import numpy as np
import torch

from ..kernels.loader import check, library
from ..kernels.ops import _dev, _p, _stream
from .params import SamplingParams
from .rng import uniform


def sample_rows(logits: torch.Tensor, temperature: torch.Tensor, top_k: torch.Tensor,
                top_p: torch.Tensor, draws: torch.Tensor) -> torch.Tensor:
    """logits [N, V] float32 on the device; per row: temperature (0 = greedy), top_k
    (0 = off), top_p (>= 1 or <= 0 = off), the uniform draw.  Returns int32 [N]."""
    _dev(logits, temperature, top_k, top_p, draws)
    if logits.dtype != torch.float32:
        raise ValueError("sampling reads float32 logits")
    N, V = logits.shape
    out = torch.empty(N, dtype=torch.int32, device=logits.device)
    lib = library("sampling.cu")
    check(lib.aie_sample_rows(_p(logits), c_int(N), c_int(V), c_int(logits.stride(0)),
                              _p(temperature), _p(top_k), _p(top_p), _p(draws), _p(out), _stream()),
          "sample_rows")
    return out


class Sampler:
    """Packs per-request options for a step and launches the kernel."""

    def __init__(self, device):
        self.device = device
        self._greedy = {}          # n -> device tensors of an all-greedy step (nothing to upload)

    def sample(self, logits: torch.Tensor, params: Sequence[SamplingParams],
               draw_index: Sequence[int]) -> torch.Tensor:
        n = len(params)
        if all(p.temperature == 0 for p in params):
            g = self._greedy.get(n)
            if g is None:
                z = torch.zeros(n, dtype=torch.float32, device=self.device)
                g = (z, torch.zeros(n, dtype=torch.int32, device=self.device),
                     torch.ones(n, dtype=torch.float32, device=self.device))
                self._greedy[n] = g
            return sample_rows(logits, g[0], g[1], g[2], g[0])
        packed = np.zeros((4, n), dtype=np.float32)
        for i, (p, k) in enumerate(zip(params, draw_index)):
            packed[0, i] = p.temperature
            packed[1, i] = p.top_p if p.top_p is not None else 1.0
            packed[2, i] = uniform(p.seed, k) if p.temperature > 0 else 0.0
        ks = np.array([p.top_k or 0 for p in params], dtype=np.int32)
        packed[3] = ks.view(np.float32)
        dev = torch.from_numpy(packed).to(self.device, non_blocking=True)
        return sample_rows(logits, dev[0], dev[3].view(torch.int32), dev[1], dev[2])
