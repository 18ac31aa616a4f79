"""Trace replay: given token ids, step by step, through the engine's own model,
step function and cache.  Nothing is sampled.  The nearest thing in the
reference feeds one token at a time through `forward_with_caches`
(crates/ai-engine-runtime/tests/generation.rs:44-56)."""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence

import torch

from ..cache.manager import PagedCache
from .loading import load_model
from .step import StepEntry, StepError, StepRunner


class Replayer:
    def __init__(self, model_dir: str, dtype: str, max_tokens: int, block_size: int = 16,
                 max_num_seqs: int = 4, device="cuda"):
        self.model, self.config = load_model(model_dir, dtype, device)
        if 64 % block_size and block_size % 64:
            raise ValueError(f"block size {block_size} must divide 64 or be a multiple of it")
        unit = max(64, block_size)
        pool_tokens = (max_tokens + unit - 1) // unit * unit
        self.cache = PagedCache(self.model.cache_requests(), page_size=block_size,
                                num_pages=pool_tokens // block_size, max_seqs=max_num_seqs,
                                max_seq_len=pool_tokens, dtype=self.model.dtype,
                                device=self.model.device)
        self.runner = StepRunner(self.model, self.cache)
        self.live: Dict[str, List[int]] = {}     # request id -> [slot, tokens in the cache]

    def run_step(self, entries: Sequence[dict], end: Sequence[str] = ()) -> Optional[torch.Tensor]:
        """Run one step; returns the wanted logits on the host (or None if no entry)."""
        batch: List[StepEntry] = []
        for e in entries:
            rid = str(e["id"])
            tokens = list(e["tokens"])
            if rid not in self.live:
                slot = self.cache.admit()
                if slot < 0:
                    raise StepError(f"request {rid}: no free slot ({self.cache.max_seqs} live requests)")
                self.live[rid] = [slot, 0]
            slot, have = self.live[rid]
            if not self.cache.ensure(slot, have + len(tokens)):
                raise StepError(f"request {rid}: the cache pool has no pages for "
                                f"{have + len(tokens)} tokens (raise --max-tokens)")
            batch.append(StepEntry(slot, have, tokens, list(e.get("want", []))))
        logits = None
        if batch:
            out = self.runner.step(batch)
            logits = out.cpu()
            self.runner.check_errors()
            for e, b in zip(entries, batch):
                st = self.live[str(e["id"])]
                st[1] += len(b.tokens)
                self.cache.advance(st[0], st[1])
        for rid in end:
            st = self.live.pop(str(rid), None)
            if st is not None:
                self.cache.finish(st[0])
        return logits
