"""The engine: model + cache + scheduler + sampler behind `generate()`.

Option names and defaults are the reference's provider keys where it has them
(crates/ai-engine-config/src/lib.rs:97-140; defaults crates/ai-engine/src/app.rs:692-703):
weights_path, device, max_num_seqs = 32, block_size = 16, kv_cache_blocks = 4096.
The loop is the reference's run_loop (crates/ai-engine-candle/src/paged/engine.rs:62-180)
with four changes: prompts are cut into portions under `max_num_batched_tokens`
and batched with decoded tokens; a request that cannot get pages is preempted and
recomputed later instead of failed; the engine is stepped by its caller rather
than by a thread of its own; and the host runs one step ahead of the device
(`async_scheduling`): step n + 1 is planned and launched while step n runs, its
decoded tokens taken from the ids that step n's sampler left on the device, and
step n's tokens are read (one pinned copy, one event) only then.  An EOS is
therefore seen one step late: the token computed past it is dropped.
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field, fields
from typing import Deque, Dict, List, Optional, Sequence, Tuple, Union

import torch

from ..cache.manager import PagedCache, host
from ..sampling.params import SamplingParams
from ..sampling.sampler import Sampler
from .loading import load_model, parse_dtype, random_model
from .step import StepEntry, StepRunner


@dataclass
class EngineOptions:
    weights_path: Optional[str] = None      # model folder (config.json + *.safetensors)
    device: str = "cuda:0"
    dtype: str = "bf16"                     # bf16 | fp32
    max_num_seqs: int = 32
    block_size: int = 16
    kv_cache_blocks: int = 4096
    kv_cache_gb: Optional[float] = None     # sizes kv_cache_blocks from a memory budget
    max_num_batched_tokens: int = 2048
    max_seq_len: Optional[int] = None       # default: max_position_embeddings
    random_weights: bool = False            # draw weights from `seed` instead of reading a folder
    seed: int = 0
    norm_weight_std: float = 0.0
    async_scheduling: bool = True           # launch step n + 1 before reading step n's tokens

    @classmethod
    def from_dict(cls, d: dict) -> "EngineOptions":
        known = {f.name for f in fields(cls)}
        unknown = sorted(set(d) - known)
        if unknown:
            raise ValueError(f"unknown engine option(s) {unknown}; known: {sorted(known)}")
        return cls(**d)

    def validate(self) -> None:
        dev = self.device
        if dev in ("auto", "cuda"):
            dev = "cuda:0"
        if dev != "cuda:0":
            raise ValueError(f"device `{self.device}` is not supported: this engine runs on cuda:0 only "
                             f"(the reference's cpu, metal and cuda:N for N > 0 are not built)")
        parse_dtype(self.dtype)
        for k in ("max_num_seqs", "block_size", "kv_cache_blocks", "max_num_batched_tokens"):
            if getattr(self, k) < 1:
                raise ValueError(f"{k} must be >= 1, got {getattr(self, k)}")


@dataclass
class _Request:
    rid: int
    tokens: List[int]               # prompt + sampled so far
    prompt_len: int
    params: SamplingParams
    output: List[int] = field(default_factory=list)
    finished: bool = False
    reason: str = ""
    pending: Optional[int] = None   # its last token is still on the device: row of the last step's sampled ids
    pending_in: object = None       # ... and the record of the step that sampled it


@dataclass
class _InFlight:
    """A launched step whose sampled ids have not been read yet."""
    items: list                     # (request, place of the token in request.tokens, finished by length)
    ids_host: Optional[torch.Tensor]        # pinned: n sampled ids, then the device error word
    event: Optional[torch.cuda.Event]


class Engine:
    def __init__(self, model: Union[str, dict, None] = None, **options):
        """model: a model folder, or a configuration (dict in config.json's keys) for
        random weights.  options: the fields of EngineOptions."""
        opts = EngineOptions.from_dict(options)
        if isinstance(model, str):
            opts.weights_path = model
        opts.validate()
        self.options = opts
        if isinstance(model, dict) or opts.random_weights:
            raw = model if isinstance(model, dict) else None
            if raw is None:
                from ..config.base import read_json
                raw = read_json(opts.weights_path)
            self.model, self.config = random_model(raw, opts.seed, opts.dtype, "cuda:0",
                                                   norm_std=opts.norm_weight_std)
        else:
            if not opts.weights_path:
                raise ValueError("Engine needs a model folder (weights_path) or a configuration")
            self.model, self.config = load_model(opts.weights_path, opts.dtype, "cuda:0")
        spec = self.model.spec
        self.max_seq_len = opts.max_seq_len or spec.max_position
        requests = self.model.cache_requests()
        blocks = opts.kv_cache_blocks
        if opts.kv_cache_gb is not None:
            probe = PagedCache(requests, opts.block_size, 1, 1, opts.block_size, self.model.dtype,
                               allocate=False)
            per_page = max(1, probe.kv_bytes_per_token() * opts.block_size)
            blocks = max(1, int(opts.kv_cache_gb * (1 << 30)) // per_page)
        self.cache = PagedCache(requests, opts.block_size, blocks, opts.max_num_seqs,
                                self.max_seq_len, self.model.dtype, self.model.device)
        self.scheduler = host().Scheduler(self.cache.book, opts.max_num_seqs,
                                          opts.max_num_batched_tokens, self.max_seq_len)
        self.runner = StepRunner(self.model, self.cache)
        self.sampler = Sampler(self.model.device)
        self.eos_ids = set(spec.eos_token_ids)
        self.requests: Dict[int, _Request] = {}
        self._next_id = 0
        self._inflight: Deque[_InFlight] = deque()
        self._pinned = [torch.zeros(opts.max_num_seqs + 1, dtype=torch.int32).pin_memory() for _ in range(3)]
        self._turn = 0
        self.counters = dict(steps=0, h2d_bytes=0, d2h_bytes=0, batch_tokens=0, batch_requests=0)

    # -- requests ------------------------------------------------------------------
    def add_request(self, prompt_ids: Sequence[int], sampling: Optional[SamplingParams] = None,
                    request_id: Optional[int] = None) -> int:
        params = sampling or SamplingParams()
        params.validate()
        rid = self._next_id if request_id is None else int(request_id)
        self._next_id = max(self._next_id, rid) + 1
        prompt = [int(t) for t in prompt_ids]
        vocab = self.model.spec.vocab_size
        bad = [t for t in prompt if not 0 <= t < vocab]
        if bad:
            raise ValueError(f"prompt holds token ids outside the vocabulary [0, {vocab}): {bad[:5]}")
        why = self.scheduler.add(rid, len(prompt), params.max_tokens)
        if why:
            raise ValueError(f"request {rid} rejected: {why}")
        self.requests[rid] = _Request(rid, prompt, len(prompt), params)
        return rid

    def has_unfinished(self) -> bool:
        return self.scheduler.has_work()

    # -- one scheduler iteration ------------------------------------------------------
    def step(self) -> List[Tuple[int, Optional[int], bool]]:
        """Schedule, run one batch, sample.  Returns (request id, token or None, finished)
        for every request whose token was read (or that ended) during this call: with
        `async_scheduling` these are the tokens of the step before the one launched here.  An EOS
        token ends its request and is not returned (crates/ai-engine-candle/src/paged/engine.rs:165-170)."""
        events: List[Tuple[int, Optional[int], bool]] = []
        plan = self.scheduler.schedule()
        for rid in plan.admitted:
            self.cache.reset_state(self.scheduler.slot(rid))
        if not plan.entries:
            self._drain(events)
            return events
        # A token that is still on the device can be handed to a lone decoded token of the next step;
        # anything else that needs it (a request preempted and recomputed) waits for the host to read it.
        for e in plan.entries:
            req = self.requests[e.id]
            if req.pending is not None and e.start + e.n_tokens == len(req.tokens) and e.n_tokens != 1:
                self._drain(events)
                break
        entries, sampled = [], []
        for e in plan.entries:
            req = self.requests.get(e.id)
            if req is None or req.finished:       # ended by an EOS that was read just now: its entry is dropped
                continue
            toks = req.tokens[e.start:e.start + e.n_tokens]
            src = req.pending if (req.pending is not None and e.start + e.n_tokens == len(req.tokens)) else None
            entries.append(StepEntry(e.slot, e.start, toks, [e.n_tokens - 1] if e.sample else [], src))
            if e.sample:
                sampled.append(req)
        if not entries:
            self.scheduler.commit(plan)
            return events
        logits = self.runner.step(entries)
        ctx = self.runner.last_ctx
        rec = _InFlight([], None, None)
        if sampled:
            n = len(sampled)
            ids = self.sampler.sample(logits, [r.params for r in sampled],
                                      [len(r.tokens) - r.prompt_len for r in sampled])
            self.runner.publish_sampled(ids)
            host = self._pinned[self._turn]
            self._turn = (self._turn + 1) % len(self._pinned)
            host[:n].copy_(ids, non_blocking=True)                 # the step's result: one read,
            host[n:n + 1].copy_(self.runner.err, non_blocking=True)   # and the device error word beside it
            rec.ids_host = host
            rec.event = torch.cuda.Event()
            rec.event.record()
            self.counters["d2h_bytes"] += (n + 1) * 4
        self.scheduler.commit(plan)
        for k, req in enumerate(sampled):
            req.tokens.append(0)                  # its place; the id is written when the step's result is read
            req.pending, req.pending_in = k, rec
            done = self.scheduler.on_token(req.rid, False)
            rec.items.append((req, len(req.tokens) - 1, done))
        self._inflight.append(rec)
        c = self.counters
        c["steps"] += 1
        c["h2d_bytes"] += ctx.h2d_bytes + (16 * len(sampled) if sampled else 0)
        c["batch_tokens"] += ctx.real_T
        c["batch_requests"] += ctx.real_R
        ahead = 1 if (self.options.async_scheduling and self.scheduler.has_work()) else 0
        while len(self._inflight) > ahead:
            self._resolve(self._inflight.popleft(), events)
        return events

    def _drain(self, events) -> None:
        while self._inflight:
            self._resolve(self._inflight.popleft(), events)

    def _resolve(self, rec: _InFlight, events) -> None:
        """Read a launched step's sampled ids and finish what they finish."""
        if rec.ids_host is None:
            return
        rec.event.synchronize()
        n = len(rec.items)
        got = rec.ids_host[:n + 1].tolist()
        if got[n]:
            self.runner.check_errors()            # raises with the meaning of the bits
        for (req, place, done), tok in zip(rec.items, got):
            if req.pending_in is rec:
                req.pending, req.pending_in = None, None
            if req.finished:                      # a token computed past an EOS: dropped
                continue
            req.tokens[place] = tok
            is_eos = tok in self.eos_ids and not req.params.ignore_eos
            if is_eos:
                del req.tokens[place + 1:]
                req.pending, req.pending_in = None, None
                if not done:
                    self.scheduler.finish(req.rid)
                done = True
            else:
                req.output.append(tok)
            if done:
                req.finished = True
                req.reason = "eos" if is_eos else "length"
            events.append((req.rid, None if is_eos else tok, done))

    # -- the call a user makes -----------------------------------------------------------
    def generate(self, prompts: Sequence[Sequence[int]],
                 sampling: Union[SamplingParams, Sequence[SamplingParams], None] = None) -> List[List[int]]:
        """Token ids in, generated token ids out (one list per prompt)."""
        if sampling is None or isinstance(sampling, SamplingParams):
            sampling = [sampling or SamplingParams()] * len(prompts)
        if len(sampling) != len(prompts):
            raise ValueError("one SamplingParams per prompt (or one for all)")
        rids = [self.add_request(p, s) for p, s in zip(prompts, sampling)]
        while self.scheduler.has_work() or self._inflight:
            self.step()
        self.runner.check_errors()
        return [self.requests.pop(r).output for r in rids]

    def take(self, request_id: int) -> List[int]:
        """The generated ids of a finished request, which the engine then forgets (callers that drive
        `add_request` / `step` themselves call this once a request's `finished` event has come)."""
        req = self.requests.get(request_id)
        if req is None or not req.finished:
            raise KeyError(f"request {request_id} is unknown or still running")
        return self.requests.pop(request_id).output

    def forward_tokens(self, entries: Sequence[StepEntry]) -> torch.Tensor:
        """The raw step function (tests, replay): logits at the wanted rows."""
        return self.runner.step(entries)

    def stats(self) -> dict:
        d = dict(self.counters)
        d.update(self.scheduler.stats())
        d["cache"] = self.cache.stats()
        d["running"] = self.scheduler.num_running
        d["waiting"] = self.scheduler.num_waiting
        return d
