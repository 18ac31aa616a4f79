"""The engine: model + cache + scheduler + sampler behind `generate()`.

Option names and defaults are the reference's provider keys where it has them
(crates/ai-engine-config/src/lib.rs:97-140; defaults crates/ai-engine/src/app.rs:692-703):
weights_path, device, max_num_seqs = 32, block_size = 16, kv_cache_blocks = 4096.
The loop is the reference's run_loop (crates/ai-engine-candle/src/paged/engine.rs:62-180)
with three changes: prompts are cut into portions under `max_num_batched_tokens`
and batched with decoded tokens; a request that cannot get pages is preempted and
recomputed later instead of failed; the engine is stepped by its caller rather
than by a thread of its own.
"""
from __future__ import annotations

from dataclasses import dataclass, field, fields
from typing import Dict, List, Optional, Sequence, Tuple, Union

import torch

from ..cache.manager import PagedCache, host
from ..config.registry import load_config
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
        self._since_check = 0
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
        for every request that got a token (or ended) in this step.  An EOS token ends
        its request and is not returned (crates/ai-engine-candle/src/paged/engine.rs:165-170)."""
        plan = self.scheduler.schedule()
        for rid in plan.admitted:
            self.cache.reset_state(self.scheduler.slot(rid))
        if not plan.entries:
            return []
        entries, sampled = [], []
        for e in plan.entries:
            req = self.requests[e.id]
            toks = req.tokens[e.start:e.start + e.n_tokens]
            entries.append(StepEntry(e.slot, e.start, toks, [e.n_tokens - 1] if e.sample else []))
            if e.sample:
                sampled.append(req)
        logits = self.runner.step(entries)
        ctx = self.runner.last_ctx
        events: List[Tuple[int, Optional[int], bool]] = []
        tokens: List[int] = []
        if sampled:
            ids = self.sampler.sample(logits, [r.params for r in sampled],
                                      [len(r.tokens) - r.prompt_len for r in sampled])
            tokens = ids.cpu().tolist()                 # the step's result: one read
            self.counters["d2h_bytes"] += len(tokens) * 4
        # the device error word is read when nothing else is (no tokens), every 16th step, and
        # whenever a request is about to end
        self._since_check += 1
        ending = any(len(r.tokens) - r.prompt_len + 1 >= r.params.max_tokens for r in sampled)
        if not sampled or ending or self._since_check >= 16:
            self.runner.check_errors()
            self._since_check = 0
            self.counters["d2h_bytes"] += 4
        self.scheduler.commit(plan)
        for req, tok in zip(sampled, tokens):
            is_eos = tok in self.eos_ids and not req.params.ignore_eos
            req.tokens.append(tok)
            done = self.scheduler.on_token(req.rid, is_eos)
            if not is_eos:
                req.output.append(tok)
            if done:
                req.finished = True
                req.reason = "eos" if is_eos else "length"
            events.append((req.rid, None if is_eos else tok, done))
        c = self.counters
        c["steps"] += 1
        c["h2d_bytes"] += ctx.h2d_bytes + (16 * len(sampled) if sampled else 0)
        c["batch_tokens"] += ctx.T
        c["batch_requests"] += ctx.R
        return events

    # -- the call a user makes -----------------------------------------------------------
    def generate(self, prompts: Sequence[Sequence[int]],
                 sampling: Union[SamplingParams, Sequence[SamplingParams], None] = None) -> List[List[int]]:
        """Token ids in, generated token ids out (one list per prompt)."""
        if sampling is None or isinstance(sampling, SamplingParams):
            sampling = [sampling or SamplingParams()] * len(prompts)
        if len(sampling) != len(prompts):
            raise ValueError("one SamplingParams per prompt (or one for all)")
        rids = [self.add_request(p, s) for p, s in zip(prompts, sampling)]
        while self.scheduler.has_work():
            self.step()
        self.runner.check_errors()
        return [self.requests.pop(r).output for r in rids]

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
