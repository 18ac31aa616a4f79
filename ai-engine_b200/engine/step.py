"""The step function: one batch of (request, its next tokens) through the model.

The reference has two functions, a whole prompt alone
(crates/ai-engine-candle/src/paged/transformer.rs:120-212) or one token for each
of B rows (:219-307).  Here there is one: every entry brings `tokens` that
follow the `start` tokens its request already has in the cache — a portion of a
prompt of any length, or one decoded token — and all entries run as one
flattened batch.  The new keys and values are written first and then read with
the mask j <= position (crates/ai-engine-runtime/src/arch/attention.rs:143-155),
which is what makes portions of prompts correct with no code of their own.
Logits come back only for the rows that are wanted.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional, Sequence

import numpy as np
import torch


@dataclass
class StepEntry:
    slot: int                    # the request's slot in the cache
    start: int                   # tokens of the request already in the cache
    tokens: Sequence[int]        # its next tokens
    want: Sequence[int] = ()     # places among `tokens` whose logits are wanted


class StepError(RuntimeError):
    pass


_ERR_BITS = {1: "a token id outside the vocabulary", 2: "a block table entry outside the page pool",
             4: "a bounded wait in a kernel ran out", 8: "a request row outside its table"}


class StepContext:
    """Device-side description of one step.  All index arrays are int32 and live
    in one buffer that is filled on the host and copied once."""

    def __init__(self, entries: Sequence[StepEntry], cache, device, err: torch.Tensor):
        R = len(entries)
        q_len = np.array([len(e.tokens) for e in entries], dtype=np.int32)
        if R == 0 or int(q_len.min()) < 1:
            raise StepError("a step needs at least one entry and every entry at least one token")
        T = int(q_len.sum())
        ctx_len = np.array([e.start for e in entries], dtype=np.int32)
        slots = np.array([e.slot for e in entries], dtype=np.int32)
        q_start = np.zeros(R, dtype=np.int32)
        np.cumsum(q_len[:-1], out=q_start[1:])
        token_ids = np.concatenate([np.asarray(e.tokens, dtype=np.int64) for e in entries])
        if token_ids.min() < 0 or token_ids.max() > 2**31 - 1:
            raise StepError("token ids must be non-negative 32-bit integers")
        token_req = np.repeat(np.arange(R, dtype=np.int32), q_len)
        positions = (np.arange(T, dtype=np.int32) - np.repeat(q_start, q_len)
                     + np.repeat(ctx_len, q_len)).astype(np.int32)
        rows: List[int] = []
        for r, e in enumerate(entries):
            for w in e.want:
                if not 0 <= w < len(e.tokens):
                    raise StepError(f"wanted place {w} is outside the entry's {len(e.tokens)} tokens")
                rows.append(int(q_start[r]) + int(w))
        N = len(rows)
        self.T, self.R, self.num_logit_rows = T, R, N
        self.h_q_len, self.h_ctx_len, self.h_slots, self.h_q_start = q_len, ctx_len, slots, q_start
        self.max_q_len = int(q_len.max())
        self.max_total_len = int((ctx_len + q_len).max())
        width = cache.block_table_width(self.max_total_len)
        tables = cache.fill_block_tables(slots.tolist(), width)

        def pad4(n):
            return (n + 3) // 4 * 4

        # requests that bring one token (decode) and the tokens of all others
        dec = q_start[q_len == 1]
        other = np.nonzero(np.repeat(q_len != 1, q_len))[0].astype(np.int32)
        self.n_decode = int(dec.shape[0])
        self.max_decode_len = int((ctx_len[q_len == 1] + 1).max()) if self.n_decode else 0
        tiles = [(r, o) for r in range(R) if q_len[r] != 1 for o in range(0, int(q_len[r]), 64)]
        segs = [("token_ids", token_ids.astype(np.int32)), ("positions", positions),
                ("decode_tokens", dec.astype(np.int32)), ("other_tokens", other),
                ("prefill_tiles", np.asarray(tiles, dtype=np.int32).reshape(-1)),
                ("token_req", token_req), ("q_start", q_start), ("q_len", q_len),
                ("ctx_len", ctx_len), ("slots", slots),
                ("logit_rows", np.asarray(rows, dtype=np.int32))]
        for g, tb in enumerate(tables):
            segs.append((f"bt{g}", tb.reshape(-1)))
        total = sum(pad4(len(a)) for _, a in segs)
        pinned = device.type == "cuda"
        host = torch.zeros(total, dtype=torch.int32, pin_memory=pinned)
        hv = host.numpy()
        offs, o = {}, 0
        for name, a in segs:
            hv[o:o + len(a)] = a
            offs[name] = (o, len(a))
            o += pad4(len(a))
        self.h2d_bytes = total * 4
        dev = host.to(device, non_blocking=True)
        self._host_keepalive = host

        def seg(name):
            b, n = offs[name]
            return dev[b:b + n]

        self.token_ids, self.positions, self.token_req = seg("token_ids"), seg("positions"), seg("token_req")
        self.q_start, self.q_len, self.ctx_len, self.slots = seg("q_start"), seg("q_len"), seg("ctx_len"), seg("slots")
        self.logit_rows = seg("logit_rows")
        self.decode_tokens, self.other_tokens = seg("decode_tokens"), seg("other_tokens")
        self.prefill_tiles = seg("prefill_tiles").view(-1, 2)
        self.block_tables = [seg(f"bt{g}").view(R, width) for g in range(len(tables))]
        self.err = err
        self.device = device


class StepRunner:
    """Binds a model to its cache and runs steps."""

    def __init__(self, model, cache):
        self.model, self.cache = model, cache
        self.device = model.device
        self.err = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.last_ctx: Optional[StepContext] = None

    def step(self, entries: Sequence[StepEntry]) -> torch.Tensor:
        """Run the entries as one batch; float32 logits [wanted rows, vocab] on the
        device, in the order of the entries and of their `want`."""
        max_len = self.cache.max_seq_len
        for e in entries:
            if e.start + len(e.tokens) > max_len:
                raise StepError(f"request in slot {e.slot} would hold {e.start + len(e.tokens)} "
                                f"tokens, more than max_seq_len {max_len}")
        ctx = StepContext(entries, self.cache, self.device, self.err)
        self.last_ctx = ctx
        return self.model.forward(ctx, self.cache)

    def check_errors(self) -> None:
        """Raise if a kernel flagged a fault since the last check (synchronises)."""
        word = int(self.err.item()) & 0xFFFFFFFF
        if word:
            self.err.zero_()
            what = [msg for bit, msg in _ERR_BITS.items() if word & bit]
            raise StepError("device error word set: " + "; ".join(what or [hex(word)]))
