"""Sampling options of a request, in the reference's names
(crates/ai-engine-runtime/src/sample.rs:4-10: temperature, top_p, top_k, seed;
max_tokens default 256 as in crates/ai-engine-candle/src/provider.rs:142-145)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional


@dataclass
class SamplingParams:
    temperature: float = 0.0          # 0 = greedy (argmax, the first maximum wins)
    top_k: Optional[int] = None       # keep the k most likely; None = off
    top_p: Optional[float] = None     # keep the shortest prefix with mass >= p; None = off
    seed: int = 42                    # the paged engine's fixed seed (paged/engine.rs:58-60)
    max_tokens: int = 256
    ignore_eos: bool = False          # keep generating past EOS (fixed-length measurement)

    def validate(self) -> None:
        if self.temperature < 0:
            raise ValueError(f"temperature must be >= 0, got {self.temperature}")
        if self.top_k is not None and self.top_k < 1:
            raise ValueError(f"top_k must be >= 1, got {self.top_k}")
        if self.top_p is not None and not 0.0 < self.top_p <= 1.0:
            raise ValueError(f"top_p must be in (0, 1], got {self.top_p}")
        if self.max_tokens < 1:
            raise ValueError(f"max_tokens must be >= 1, got {self.max_tokens}")
