"""Runs the sampling kernel over the rows of a step's logits."""
from __future__ import annotations

from ctypes import c_int
from typing import Sequence

import numpy as np
import torch

from ..kernels.loader import check, library
from ..kernels.ops import _dev, _nb, _p, _stream
from ..kernels.profile import region
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
    with region("sample_rows", _nb(logits)):
        check(lib.aie_sample_rows(_p(logits), c_int(N), c_int(V), c_int(logits.stride(0)),
                                  _p(temperature), _p(top_k), _p(top_p), _p(draws), _p(out), _stream()),
              "sample_rows")
    return out


def argmax_rows(logits: torch.Tensor, scratch) -> torch.Tensor:
    """Greedy for every row: int32 [N], the first maximum.  scratch: (int64 [>= N], int32 [>= N]) zeroed
    device tensors that the kernel leaves zeroed (a row is spread over several blocks)."""
    _dev(*scratch)
    if logits.dtype != torch.float32 or not logits.is_cuda or logits.dim() != 2 or logits.stride(1) != 1:
        raise ValueError("sampling reads float32 logits [N, V] on the device, rows contiguous")
    N, V = logits.shape
    out = torch.empty(N, dtype=torch.int32, device=logits.device)
    lib = library("sampling.cu")
    with region("argmax_rows", _nb(logits)):
        check(lib.aie_argmax_rows(_p(logits), c_int(N), c_int(V), c_int(logits.stride(0)), _p(scratch[0]), _p(scratch[1]),
                                  _p(out), _stream()), "argmax_rows")
    return out


class Sampler:
    """Packs per-request options for a step and launches the kernel."""

    def __init__(self, device):
        self.device = device
        self._scratch = None       # zeroed scratch of the all-greedy kernel

    def sample(self, logits: torch.Tensor, params: Sequence[SamplingParams],
               draw_index: Sequence[int]) -> torch.Tensor:
        n = len(params)
        if all(p.temperature == 0 for p in params):
            if self._scratch is None or self._scratch[0].shape[0] < n:
                m = max(n, 64)
                self._scratch = (torch.zeros(m, dtype=torch.int64, device=self.device),
                                 torch.zeros(m, dtype=torch.int32, device=self.device))
            return argmax_rows(logits, self._scratch)
        packed = np.zeros((4, n), dtype=np.float32)
        for i, (p, k) in enumerate(zip(params, draw_index)):
            packed[0, i] = p.temperature
            packed[1, i] = p.top_p if p.top_p is not None else 1.0
            packed[2, i] = uniform(p.seed, k) if p.temperature > 0 else 0.0
        ks = np.array([p.top_k or 0 for p in params], dtype=np.int32)
        packed[3] = ks.view(np.float32)
        dev = torch.from_numpy(packed).to(self.device, non_blocking=True)
        return sample_rows(logits, dev[0], dev[3].view(torch.int32), dev[1], dev[2])
