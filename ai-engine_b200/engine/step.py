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

import os
from dataclasses import dataclass
from types import SimpleNamespace
from typing import List, Optional, Sequence

import numpy as np
import torch



@dataclass
class StepEntry:
    slot: int                    # the request's slot in the cache
    start: int                   # tokens of the request already in the cache
    tokens: Sequence[int]        # its next tokens
    want: Sequence[int] = ()     # places among `tokens` whose logits are wanted
    src: Optional[int] = None    # its one token is still on the device: row of the previous step's sampled ids


class StepError(RuntimeError):
    pass


_ERR_BITS = {1: "a token id outside the vocabulary", 2: "a block table entry outside the page pool",
             4: "a bounded wait in a kernel ran out", 8: "a request row outside its table"}


class _Staging:
    """A ring of pinned host buffers shared by all layouts: the host may run ahead of the device, so a
    buffer is rewritten only after the copy that read it has finished.  They grow with the largest step
    (pinning memory takes about half a millisecond: not once per layout)."""

    def __init__(self, pinned: bool, depth: int = 4):
        self.pinned = pinned
        self.hosts = [None] * depth
        self.copied = [None] * depth
        self.turn = 0

    def take(self, n: int):
        """(index, int32 host view of n elements) of the next buffer, free to be written."""
        i = self.turn
        self.turn = (i + 1) % len(self.hosts)
        if self.copied[i] is not None:
            self.copied[i].synchronize()
        h = self.hosts[i]
        if h is None or h.shape[0] < n:
            h = torch.zeros(max(1024, 1 << (n - 1).bit_length()), dtype=torch.int32, pin_memory=self.pinned)
            self.hosts[i] = h
        return i, h[:n]

    def sent(self, i: int) -> None:
        if self.pinned:
            ev = self.copied[i] or torch.cuda.Event()
            ev.record()
            self.copied[i] = ev


class _Buffers:
    """The device int32 buffer of one layout (one tuple of segment lengths), reused by every step
    of that layout; a CUDA graph captured on it stays valid because its address never changes."""

    def __init__(self, lengths, device, staging: Optional[_Staging] = None):
        self.offsets, o = [], 0
        for n in lengths:
            self.offsets.append((o, n))
            o += (n + 3) // 4 * 4
        self.total = max(o, 4)
        self.staging = staging or _Staging(device.type == "cuda")
        self.dev = torch.zeros(self.total, dtype=torch.int32, device=device)
        self.graph = None          # torch.cuda.CUDAGraph of a decode-only step on these buffers
        self.graph_logits = None
        self.graph_kernels = 0
        self.uses = 0
        self.views = None          # device views of the segments, made at the layout's first step

    def upload(self, arrays) -> None:
        i, host = self.staging.take(self.total)
        hv = host.numpy()
        for (o, n), a in zip(self.offsets, arrays):
            hv[o:o + n] = a
        self.dev.copy_(host, non_blocking=True)
        self.staging.sent(i)


class StepContext:
    """Device-side description of one step.  All index arrays are int32 and live in one buffer that
    is filled on the host and copied once.

    Generic arrays (what any part may read): `token_ids`, `positions`, `token_req` [T] (row of the token's
    request); `q_start`, `q_len`, `ctx_len`, `slots`, `live` [R] (first token, tokens brought, tokens already
    cached, cache slot, 0 for a row that only rounds the batch up); `logit_rows` [N]; `token_src` [T];
    one block table [R, bt_width] per cache group.  Their host copies are `h_q_start`, `h_q_len`,
    `h_ctx_len`, `h_slots`.  Lists that only one kind of part wants are made by that part's
    `StepPlanner` and read with `plan(planner)`."""

    SEGMENTS = ("token_ids", "positions", "token_req", "q_start", "q_len", "ctx_len", "slots", "live",
                "logit_rows", "token_src")

    def __init__(self, entries: Sequence[StepEntry], cache, device, err: torch.Tensor,
                 buffers: Optional[dict] = None, bucket_width: bool = False, planners=(),
                 n_live: Optional[int] = None):
        # The generic arrays and the block tables are packed by the host runtime (csrc/host/step_pack.hpp) into one
        # int32 array; what the planners add goes behind it.
        from ..cache.manager import host as host_runtime

        try:
            packed, lengths, T, R, N, max_q, max_total, width, has_src = host_runtime().pack_step(
                cache.book, [e.slot for e in entries], [e.start for e in entries], [e.tokens for e in entries],
                [e.want for e in entries], [-1 if e.src is None else e.src for e in entries],
                -1 if n_live is None else int(n_live), cache.page_size, bool(bucket_width))
        except ValueError as e:
            raise StepError(str(e)) from None
        self.T, self.R, self.num_logit_rows, self.has_src = T, R, N, has_src
        self.max_q_len, self.max_total_len = max_q, max_total
        self.bt_width, self.page_size, self.bucketed = width, cache.page_size, bool(bucket_width)
        offs, o = [], 0
        for n in lengths:
            offs.append((o, n))
            o += (n + 3) // 4 * 4
        host = [packed[o:o + n] for o, n in offs]
        self.h_q_start, self.h_q_len, self.h_ctx_len, self.h_slots = host[3], host[4], host[5], host[6]

        arrays = [packed]
        planned = []                # (planner, [(name, shape)], scalars)
        for pl in planners:
            arrs, scalars = pl.plan(self)
            planned.append((pl, [(name, a.shape) for name, a in arrs.items()], scalars))
            arrays += [np.ascontiguousarray(a, dtype=np.int32).reshape(-1) for a in arrs.values()]
        key = tuple(lengths) + tuple(len(a) for a in arrays[1:]) + (width,) + tuple(pl.key for pl in planners)
        self.layout_key = key
        buf = buffers.get(key) if buffers is not None else None
        if buf is None:
            buf = _Buffers([len(a) for a in arrays], device, buffers.get("staging") if buffers is not None else None)
            if buffers is not None:
                if len(buffers) >= 128:
                    buffers.pop(next(k for k in buffers if k != "staging"))
                buffers[key] = buf
        buf.uses += 1
        self.buffers = buf
        buf.upload(arrays)
        self.h2d_bytes = buf.total * 4
        if buf.views is None:       # the device views of a layout are made once: its offsets never change
            dev = buf.dev
            generic = [dev[o:o + n] for o, n in offs]
            buf.views = (generic[:10], [v.view(R, width) for v in generic[10:]],
                         [dev[o:o + n] for o, n in buf.offsets[1:]])
        generic, self.block_tables, views = buf.views
        (self.token_ids, self.positions, self.token_req, self.q_start, self.q_len, self.ctx_len, self.slots,
         self.live, self.logit_rows, self.token_src) = generic
        self._plans = {}
        at = 0
        for pl, shapes, scalars in planned:
            ns = SimpleNamespace(**scalars)
            for name, shape in shapes:
                setattr(ns, name, views[at] if len(shape) == 1 else views[at].view(shape))
                at += 1
            self._plans[id(pl)] = ns
        self.err = err
        self.device = device

    def plan(self, planner):
        """The lists of `planner` for this step.  They are in the step's buffer when the planner was known
        when the step was built (`StepRunner` passes its model's planners); else they are made and uploaded
        now, each by a copy of its own."""
        ns = self._plans.get(id(planner))
        if ns is None:
            arrs, scalars = planner.plan(self)
            ns = SimpleNamespace(**scalars)
            for name, a in arrs.items():
                setattr(ns, name, torch.from_numpy(np.ascontiguousarray(a, dtype=np.int32)).to(self.device))
            self._plans[id(planner)] = ns
        return ns


class StepRunner:
    """Binds a model to its cache and runs steps.  Steps in which every request
    brings one token (decode) are captured once per layout as a CUDA graph and
    replayed: the launch cost of some hundred kernels a step is paid once."""

    def __init__(self, model, cache, use_graphs: Optional[bool] = None, capture_at_use: int = 2):
        """capture_at_use: a decode layout is captured at this use of it (2: a layout seen once is not worth a
        capture; batches rounded up to a multiple of 8 and block-table widths in powers of two keep layouts few)."""
        self.model, self.cache = model, cache
        self.capture_at_use = max(1, int(capture_at_use))
        self.device = model.device
        self.err = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.last_ctx: Optional[StepContext] = None
        self.buffers: dict = {"staging": _Staging(self.device.type == "cuda")}
        if use_graphs is None:
            from ..kernels import profile
            use_graphs = (model.dtype == torch.bfloat16 and not model.has_host_parts()
                          and not os.environ.get("AI_ENGINE_B200_NO_GRAPHS") and not profile.enabled())
        self.use_graphs = bool(use_graphs) and self.device.type == "cuda"
        # decode steps are rounded up by repeating a row only if every part that keeps state skips such rows
        self.pad_decode = model.pads_decode_rows() if hasattr(model, "pads_decode_rows") else True
        self.planners = tuple(model.step_planners()) if hasattr(model, "step_planners") else ()
        self.graph_launches = 0        # kernels replayed through graphs (for launch counts)
        self.graphs_captured = 0
        # the ids the last step sampled, left on the device for a next step that starts before the
        # host has read them (StepEntry.src)
        self.sampled = torch.zeros(max(1, getattr(cache, 'max_seqs', 1)), dtype=torch.int32, device=self.device)

    def publish_sampled(self, ids: torch.Tensor) -> None:
        """Keep this step's sampled ids (int32 [n], on the device) for the next step's entries with `src`."""
        self.sampled[:ids.shape[0]].copy_(ids)

    def step(self, entries: Sequence[StepEntry]) -> torch.Tensor:
        """Run the entries as one batch; float32 logits [wanted rows, vocab] on the
        device, in the order of the entries and of their `want`.  The tensor is
        valid until the next call of step()."""
        max_len = self.cache.max_seq_len
        decode_only = True
        for e in entries:
            if e.start + len(e.tokens) > max_len:
                raise StepError(f"request in slot {e.slot} would hold {e.start + len(e.tokens)} "
                                f"tokens, more than max_seq_len {max_len}")
            decode_only = decode_only and len(e.tokens) == 1
        graphed = self.use_graphs and decode_only
        n_real, real_rows = len(entries), None
        if graphed and self.pad_decode and n_real > 8 and n_real % 8:
            # the number of requests of a decode step is rounded up to a multiple of 8 by repeating the entry
            # with the fewest cached tokens (the same token at the same place: it writes the same key and value
            # again, and reads the shortest cache), so that batches that shrink and grow request by request share
            # their layouts, and with them their graphs
            real_rows = sum(len(e.want) for e in entries)
            e0 = min(entries, key=lambda e: e.start)
            entries = list(entries) + [StepEntry(e0.slot, e0.start, e0.tokens, [0], e0.src)] * (8 - n_real % 8)
        ctx = StepContext(entries, self.cache, self.device, self.err, self.buffers, bucket_width=graphed,
                          planners=self.planners, n_live=n_real)
        ctx.real_R, ctx.real_T = n_real, ctx.T - (len(entries) - n_real)
        self.last_ctx = ctx
        if ctx.has_src:
            from ..kernels import ops
            ops.take_sampled_ids(ctx.token_ids, ctx.token_src, self.sampled, self.err)
        logits = self._run(ctx, graphed)
        return logits if real_rows is None else logits[:real_rows]

    def _run(self, ctx: StepContext, graphed: bool) -> torch.Tensor:
        if not graphed:
            return self.model.forward(ctx, self.cache)
        buf = ctx.buffers
        if buf.graph is None:
            if buf.uses < self.capture_at_use:     # a layout seen only once is not worth a capture
                return self.model.forward(ctx, self.cache)
            from ..kernels.loader import LAUNCHES
            # This step runs eagerly (which is also the warm-up that a capture needs: library set-up) and
            # its logits are the step's result; the capture that follows launches nothing, so a part that
            # keeps state is updated once.  The graph is replayed from the layout's next use on.
            logits = self.model.forward(ctx, self.cache)
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            n0 = LAUNCHES[0]
            with torch.cuda.graph(g):
                buf.graph_logits = self.model.forward(ctx, self.cache)
            buf.graph_kernels = LAUNCHES[0] - n0
            buf.graph = g
            self.graphs_captured += 1
            return logits
        buf.graph.replay()
        self.graph_launches += buf.graph_kernels
        return buf.graph_logits

    def check_errors(self) -> None:
        """Raise if a kernel flagged a fault since the last check (synchronises)."""
        word = int(self.err.item()) & 0xFFFFFFFF
        if word:
            self.err.zero_()
            what = [msg for bit, msg in _ERR_BITS.items() if word & bit]
            raise StepError("device error word set: " + "; ".join(what or [hex(word)]))
