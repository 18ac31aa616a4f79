"""Decode and prefill throughput of the engine on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

Default run: the layer sizes of Llama-3-8B (32 layers, hidden 4096, 32 heads, 8 kv
heads, head size 128, intermediate 14336, vocabulary 128256, bf16, random weights
N(0, 0.02)), 8 requests with 1,024-token prompts in the cache of an 8,192-token
context, KV page 16.  A step is one decode step of the whole batch.  Prints ONE
JSON line: `value` = decoded tokens per second on the device (CUDA events around
blocks of K steps: the median of five blocks, their spread in `spread`), `e2e` = the same
through Engine.add_request()/Engine.step() with host tokens in and out, `prefill` = one
2,048-token prompt in one step (the median of five), `roofline` = the bytes a decode
step has to read (every weight once + the live requests' cache) over its time against
the measured copy bandwidth, `points` = decode at batch 1 and 64 and at 8,192 tokens of
context, and the headline figures of the two serving workloads.

Parts alone (one line each, for profiles): `--only decode|prefill` (with `--layers`,
`--batch`), `--only gemm` (each projection at `--batch` tokens: library product and
the tcgen05 kernel), `--only attention` (the prompt-attention kernels), `--only peaks`
(a device copy and a library bf16 product on this box).  The other
configurations of the baseline through the engine's scheduler: `--workload serving1b|long3b`
(per phase: bytes a step had to read and the fraction of the copy bandwidth, prompt TFLOP/s
against the library product's peak, what the steps were made of, how often the device
waited for the host).  `--profile`: CUDA-event time per class of kernel for one prefill
step and for decode steps, launched eagerly, with bytes, flops and the fraction of the
roofline for each class.
"""
import argparse
import json
import os
import statistics
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

LLAMA3_8B = dict(architectures=["LlamaForCausalLM"], hidden_size=4096, intermediate_size=14336,
                 num_hidden_layers=32, num_attention_heads=32, num_key_value_heads=8, head_dim=128,
                 vocab_size=128256, max_position_embeddings=8192, rope_theta=500000.0,
                 rms_norm_eps=1e-5, tie_word_embeddings=False)
CONTEXT, PROMPT_LEN, PREFILL_TOKENS, PAGE = 8192, 1024, 2048, 16


def peaks():
    """Measured peaks if the driver wrote them, else the stated fallback."""
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            m = json.load(open(p))
            return dict(hbm_gbs=float(m["hbm_gbs"]), bf16_tflops=float(m["bf16_tflops"]),
                        bf16_tflops_sustained=float(m.get("bf16_tflops_sustained", m["bf16_tflops"])),
                        source="measured")
        except Exception:
            pass
    return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, bf16_tflops_sustained=1400.0, source="fallback")


class ClockSampler:
    """SM clock and throttle reasons every 100 ms while the timed region runs (read only)."""
    REASONS = {0x4: "sw_power_cap", 0x8: "hw_slowdown", 0x20: "sw_thermal_slowdown",
               0x40: "hw_thermal_slowdown", 0x80: "hw_power_brake_slowdown"}

    def __init__(self):
        self.samples, self.reasons, self.max_mhz, self._stop = [], set(), None, threading.Event()
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv, self.h = pynvml, pynvml.nvmlDeviceGetHandleByIndex(0)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def _run(self):
        while not self._stop.wait(0.1):
            try:
                self.samples.append(self.nv.nvmlDeviceGetClockInfo(self.h, self.nv.NVML_CLOCK_SM))
                r = self.nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                self.reasons |= {n for bit, n in self.REASONS.items() if r & bit}
            except Exception:
                pass

    def __enter__(self):
        if self.nv:
            self.t = threading.Thread(target=self._run, daemon=True)
            self.t.start()
        return self

    def __exit__(self, *a):
        self._stop.set()
        if self.nv:
            self.t.join()

    def summary(self):
        return dict(sm_mhz=statistics.median(self.samples) if self.samples else None,
                    sm_max_mhz=self.max_mhz, reasons=sorted(self.reasons))


def time_decode(torch, aie, model, batch, prompt_len, steps, warmup, ctx_cap, blocks=5):
    """Device time of decode steps of `batch` requests that each hold prompt_len tokens: `blocks` blocks
    of `steps` steps, each between a pair of CUDA events; the median block is the result, the fastest and
    slowest are its spread.  The cache is filled by a real prefill through the step function."""
    from ai_engine_b200.cache import PagedCache
    from ai_engine_b200.engine.step import StepEntry, StepRunner
    from ai_engine_b200.kernels.loader import LAUNCHES
    from ai_engine_b200.sampling.sampler import Sampler

    total = min(prompt_len + warmup + steps * blocks + 1, ctx_cap)
    blocks = max(1, min(blocks, (total - prompt_len - warmup - 1) // steps))
    pages = batch * ((total + PAGE - 1) // PAGE) + 4
    cache = PagedCache(model.cache_requests(), PAGE, pages, batch, ctx_cap, model.dtype, model.device)
    runner = StepRunner(model, cache)
    g = torch.Generator().manual_seed(0)
    vocab = model.spec.vocab_size
    slots = [cache.admit() for _ in range(batch)]
    for s in slots:
        assert cache.ensure(s, total)
    for s in slots:           # prefill, one request a step, in portions of 2,048 tokens
        ids = torch.randint(0, vocab, (prompt_len,), generator=g).tolist()
        for a in range(0, prompt_len, 2048):
            runner.step([StepEntry(s, a, ids[a:a + 2048], [])])
    runner.check_errors()
    sampler = Sampler(model.device)
    greedy = [aie.SamplingParams(max_tokens=1, temperature=0.0)] * batch
    tokens = torch.randint(0, vocab, (batch,), generator=g).tolist()

    def one(i):
        nonlocal tokens
        logits = runner.step([StepEntry(s, prompt_len + i, [tokens[j]], [0]) for j, s in enumerate(slots)])
        return sampler.sample(logits, greedy, [0] * batch)

    for i in range(warmup):
        out = one(i)
    tokens = out.cpu().tolist()
    torch.cuda.synchronize()
    l0, g0 = LAUNCHES[0], runner.graph_launches
    per_block = []
    for blk in range(blocks):
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for i in range(steps):
            out = one(warmup + blk * steps + i)
        end.record()
        torch.cuda.synchronize()
        per_block.append(start.elapsed_time(end) / steps)
    runner.check_errors()
    launches = (LAUNCHES[0] - l0 + runner.graph_launches - g0) // blocks     # launched afresh + replayed, per block
    ms = statistics.median(per_block)
    ctx_tokens = batch * (prompt_len + warmup + steps * blocks / 2.0)
    bytes_step = model.step_weight_bytes() + cache.kv_bytes_per_token() * ctx_tokens
    del cache, runner
    torch.cuda.empty_cache()
    return dict(ms=ms, ms_min=min(per_block), ms_max=max(per_block), blocks=blocks, tok_s=batch * 1000.0 / ms,
                launches=launches, bytes=bytes_step)


def time_e2e(torch, aie, model_cfg, batch, prompt_len, steps, warmup, layers, blocks=5):
    """Through the public API: add_request(host ids) then step() — every step copies its
    inputs from pinned host memory and reads the sampled tokens back.  Wall clock around blocks of
    `steps` calls of Engine.step(); the median block is the result."""
    eng = aie.Engine(model_cfg, dtype="bf16", random_weights=True, seed=0, max_num_seqs=batch,
                     block_size=PAGE, kv_cache_blocks=batch * ((prompt_len + steps * blocks + warmup + 32) // PAGE + 2),
                     max_num_batched_tokens=2048, max_seq_len=CONTEXT)
    g = torch.Generator().manual_seed(1)
    sp = aie.SamplingParams(max_tokens=steps * blocks + warmup + 8, ignore_eos=True)
    for _ in range(batch):
        eng.add_request(torch.randint(0, model_cfg["vocab_size"], (prompt_len,), generator=g).tolist(), sp)
    while eng.scheduler.num_waiting or any(eng.scheduler.computed(r) < prompt_len for r in eng.scheduler.running()):
        eng.step()
    for _ in range(warmup):
        eng.step()
    torch.cuda.synchronize()
    c0 = dict(eng.counters)
    rates = []
    for _ in range(blocks):
        t0 = time.perf_counter()
        n = 0
        for _ in range(steps):
            n += len(eng.step())
        torch.cuda.synchronize()
        rates.append(n / (time.perf_counter() - t0))
    c1 = eng.counters
    return dict(value=statistics.median(rates), unit="tokens/s", value_min=round(min(rates), 1), value_max=round(max(rates), 1),
                h2d_bytes_per_step=(c1["h2d_bytes"] - c0["h2d_bytes"]) // (steps * blocks),
                d2h_bytes_per_step=(c1["d2h_bytes"] - c0["d2h_bytes"]) // (steps * blocks)), eng


def time_prefill(torch, model, tokens, pk):
    from ai_engine_b200.cache import PagedCache
    from ai_engine_b200.engine.step import StepEntry, StepRunner

    cache = PagedCache(model.cache_requests(), PAGE, tokens // PAGE + 2, 1, CONTEXT, model.dtype, model.device)
    runner = StepRunner(model, cache)
    ids = torch.randint(0, model.spec.vocab_size, (tokens,), generator=torch.Generator().manual_seed(2)).tolist()
    times = []
    for it in range(7):           # two warm-up steps, then five timed ones: the median is reported
        slot = cache.admit()
        cache.ensure(slot, tokens)
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        runner.step([StepEntry(slot, 0, ids, [tokens - 1])])
        e.record()
        torch.cuda.synchronize()
        cache.finish(slot)
        if it >= 2:
            times.append(s.elapsed_time(e))
    runner.check_errors()
    best = statistics.median(times)
    flops = model.step_flops(tokens, keys=(tokens + 1) / 2.0, logit_rows=1)      # what the parts report
    return dict(value=tokens * 1000.0 / best, tokens=tokens, ms=best, ms_min=min(times), ms_max=max(times),
                frac=flops / (best * 1e-3) / (pk["bf16_tflops"] * 1e12))


def time_gemms(torch, tokens):
    """Each projection of the model alone at `tokens` rows: the library product and the
    tcgen05 kernel (with several split-K settings for small steps), L2 flushed between runs."""
    from ai_engine_b200.kernels import ops

    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    err = torch.zeros(1, dtype=torch.int32, device="cuda")
    shapes = {"qkv": (6144, 4096), "o": (4096, 4096), "gate_up": (28672, 4096), "down": (4096, 14336),
              "lm_head": (128256, 4096)}
    out = {}
    for name, (N, K) in shapes.items():
        T = 1 if name == "lm_head" and tokens > 64 else tokens
        x = torch.randn(T, K, device="cuda").bfloat16()
        w = (torch.randn(N, K, device="cuda") * 0.02).bfloat16()
        impls = {"library": lambda: torch.mm(x, w.t()), "tcgen05": lambda: ops.gemm_tc(x, w, torch.bfloat16, err)}
        for s_ in (2, 3, 4, 6, 9, 13):       # K cut into parts that are left for the consumer to add
            if T <= 64 and N < 148 * 128:
                impls[f"tcgen05_p{s_}"] = (lambda s_=s_: ops.gemm_tc(x, w, torch.float32, err, splits=s_, raw_parts=True))
        if name == "gate_up" and T <= 64:       # the activation in the epilogue, K cut into parts joined in a cluster
            for s_ in (1, 2, 3, 4):
                impls[f"tcgen05_swiglu_s{s_}"] = (lambda s_=s_: ops.gemm_tc(x, w, torch.bfloat16, err, splits=s_, swiglu=True))
        row = {}
        for iname, fn in impls.items():
            for _ in range(3):
                fn()
            ts = []
            for _ in range(10):
                flush.zero_()
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record()
                fn()
                b.record()
                torch.cuda.synchronize()
                ts.append(a.elapsed_time(b) * 1e3)
            us = sorted(ts)[len(ts) // 2]
            row[iname] = dict(us=round(us, 1), tb_s=round((N * K * 2 + T * (K + N) * 2) / us / 1e6, 2),
                              tflops=round(2.0 * T * N * K / us / 1e6, 1))
        out[f"{name}[{T}x{N}x{K}]"] = row
    assert int(err.item()) == 0
    return out


def time_peaks(torch):
    """What this box does on a plain device copy (read + write bytes over time) and on a library bf16 product:
    the two figures the roofline fractions are taken against, measured here for context (the fractions in
    the JSON line use MEASURED_PEAKS.json when the driver wrote it, else the stated fallback)."""
    out = {}
    n = 1 << 30
    a = torch.empty(n, dtype=torch.uint8, device="cuda")
    b = torch.empty_like(a)
    ts = []
    for i in range(8):
        s_, e_ = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s_.record()
        b.copy_(a)
        e_.record()
        torch.cuda.synchronize()
        if i >= 3:
            ts.append(s_.elapsed_time(e_))
    out["copy_gb_s"] = round(2 * n / (sorted(ts)[len(ts) // 2] * 1e-3) / 1e9, 1)
    del a, b
    m = 8192
    x = torch.randn(m, m, device="cuda").bfloat16()
    w = torch.randn(m, m, device="cuda").bfloat16()
    ts = []
    for i in range(8):
        s_, e_ = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s_.record()
        torch.mm(x, w.t())
        e_.record()
        torch.cuda.synchronize()
        if i >= 3:
            ts.append(s_.elapsed_time(e_))
    out["bf16_tflops_burst"] = round(2.0 * m ** 3 / (sorted(ts)[len(ts) // 2] * 1e-3) / 1e12, 1)
    s_, e_ = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s_.record()
    for _ in range(1500):
        torch.mm(x, w.t())
    e_.record()
    torch.cuda.synchronize()
    out["bf16_tflops_sustained"] = round(1500 * 2.0 * m ** 3 / (s_.elapsed_time(e_) * 1e-3) / 1e12, 1)
    return out


def time_attention(torch, tokens, context):
    """The attention kernels for a portion of `tokens` prompt tokens after `context` cached ones, alone, at the
    flagship head layout (32 heads on 8 kv heads of 128, pages of 16): the tcgen05 kernel and the mma.sync
    kernel, median of 10 with L2 flushed between runs; TFLOP/s counts the causal half only."""
    from ai_engine_b200.kernels import ops

    H, K, d, P = 32, 8, 128, 16
    total = context + tokens
    n_pages = (total + P - 1) // P
    dev = "cuda"
    torch.manual_seed(0)
    kp = (torch.randn(n_pages, K, P, d, device=dev) * 0.5).bfloat16()
    vp = torch.randn(n_pages, K, P, d, device=dev).bfloat16()
    q = torch.randn(tokens, H, d, device=dev).bfloat16()
    i32 = lambda a: torch.tensor(a, dtype=torch.int32, device=dev)
    bt = torch.randperm(n_pages, device=dev).int().view(1, -1).contiguous()
    tiles = i32([[0, o] for o in range(0, tokens, ops.PREFILL_TILE)])
    qs, ql, cl = i32([0]), i32([tokens]), i32([context])
    err = torch.zeros(1, dtype=torch.int32, device=dev)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    outs, row = {}, {}
    units = i32([[0, o] for o in range(0, tokens, 2 * ops.PREFILL_TILE)])
    impls = {"tcgen05": lambda o: ops.paged_attention_prefill_tc(q, kp, vp, tiles, qs, ql, cl, bt, d ** -0.5, 0, err, o),
             "tcgen05_pair": lambda o: ops.paged_attention_prefill_tc(q, kp, vp, units, qs, ql, cl, bt, d ** -0.5, 0, err, o,
                                                                      pair=True),
             "mma_sync": lambda o: ops.paged_attention_prefill(q, kp, vp, tiles, qs, ql, cl, bt, d ** -0.5, 0, err, o)}
    flops = 4.0 * d * H * (tokens * context + tokens * (tokens + 1) / 2)
    for name, fn in impls.items():
        outs[name] = torch.zeros_like(q)
        for _ in range(3):
            fn(outs[name])
        ts = []
        for _ in range(10):
            flush.zero_()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            fn(outs[name])
            b.record()
            torch.cuda.synchronize()
            ts.append(a.elapsed_time(b) * 1e3)
        us = sorted(ts)[len(ts) // 2]
        row[name] = dict(us=round(us, 1), tflops=round(flops / us / 1e6, 1))
    assert int(err.item()) == 0
    row["max_difference"] = float((outs["tcgen05"].float() - outs["mma_sync"].float()).abs().max())
    row["max_difference_pair"] = float((outs["tcgen05_pair"].float() - outs["mma_sync"].float()).abs().max())
    return {f"attention[{tokens} tokens after {context}]": row}


def time_decode_attention(torch, H, K, d, lens):
    """The decode attention kernels alone for one layer's lone tokens over cached contexts of `lens` tokens (pages
    of 16): the split-KV kernel with the number of parts the engine would choose, median of 10 with L2 flushed
    between runs; GB/s counts the keys and values read once."""
    from ai_engine_b200.kernels import ops

    P, dev = PAGE, "cuda"
    R = len(lens)
    pages_per = [(n + P - 1) // P for n in lens]
    n_pages = sum(pages_per) + 1
    torch.manual_seed(0)
    kp = (torch.randn(n_pages, K, P, d, device=dev) * 0.5).bfloat16()
    vp = torch.randn(n_pages, K, P, d, device=dev).bfloat16()
    q = torch.randn(R, H, d, device=dev).bfloat16()
    perm = torch.randperm(n_pages, device=dev).int()
    bt = torch.zeros((R, max(pages_per)), dtype=torch.int32, device=dev)
    at = 0
    for r, n in enumerate(pages_per):
        bt[r, :n] = perm[at:at + n]
        at += n
    i32 = lambda a: torch.tensor(a, dtype=torch.int32, device=dev)
    # lone-token rows in the order the engine lists them: longest context first
    pos, req, dec = i32([n - 1 for n in lens]), i32(list(range(R))), i32(sorted(range(R), key=lambda r: -lens[r]))
    err = torch.zeros(1, dtype=torch.int32, device=dev)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    splits = ops.decode_splits(R, K, H // K, max(lens), bt.shape[1])
    outs = {"split": torch.zeros_like(q)}
    impls = {"split": lambda: ops.paged_attention_decode(q, kp, vp, dec, pos, req, bt, d ** -0.5, 0, splits, err, outs["split"])}
    nbytes = sum(lens) * K * d * 2 * 2
    row = {}
    for name, fn in impls.items():
        for _ in range(3):
            fn()
        ts = []
        for _ in range(10):
            flush.zero_()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            fn()
            b.record()
            torch.cuda.synchronize()
            ts.append(a.elapsed_time(b) * 1e3)
        us = sorted(ts)[len(ts) // 2]
        row[name] = dict(us=round(us, 1), gb_s=round(nbytes / us / 1e3, 1))
    assert int(err.item()) == 0
    row["split_parts"] = splits
    return {f"decode attention[{R} requests, {sum(lens)} keys, H{H} K{K} d{d}]": row}


LLAMA32_1B = dict(architectures=["LlamaForCausalLM"], hidden_size=2048, intermediate_size=8192,
                  num_hidden_layers=16, num_attention_heads=32, num_key_value_heads=8, head_dim=64,
                  vocab_size=128256, max_position_embeddings=131072, rope_theta=500000.0, rms_norm_eps=1e-5,
                  tie_word_embeddings=True,
                  rope_scaling=dict(rope_type="llama3", factor=32.0, low_freq_factor=1.0, high_freq_factor=4.0,
                                    original_max_position_embeddings=8192))
LLAMA32_3B = dict(LLAMA32_1B, hidden_size=3072, num_hidden_layers=28, num_attention_heads=24, head_dim=128)


def run_workload(torch, aie, name, pk):
    """The two serving workloads of the baseline's other configurations, through the engine's scheduler
    (add_request + step, as Engine.generate() does):
    serving1b — Llama-3.2-1B shape, 64 concurrent requests, prompts uniform in [128, 4096], 256 tokens each;
    long3b    — Llama-3.2-3B shape, one 32,768-token prompt in 2,048-token portions, then 512 greedy tokens.
    Every step is put down with its time on the device (a CUDA event behind every step's launches: the host
    runs ahead of the device, through prompt portions that sample nothing by many steps, so wall-clock times
    of the calls say nothing about a step), what it was made of, the bytes it had to read (every weight once
    and the cache of its requests) and its flops; steps in which every request brings one token are the decode
    phase, the others the prompt phase."""
    g = torch.Generator().manual_seed(0)
    if name == "serving1b":
        cfg, n, new = LLAMA32_1B, 64, 256
        lens = torch.randint(128, 4097, (n,), generator=g).tolist()
        opts = dict(max_num_seqs=64, kv_cache_blocks=(sum(lens) + n * new) // PAGE + 2 * n, max_num_batched_tokens=2048,
                    max_seq_len=8192)
    else:
        cfg, n, new = LLAMA32_3B, 1, 512
        lens = [32768]
        opts = dict(max_num_seqs=1, kv_cache_blocks=(32768 + new) // PAGE + 4, max_num_batched_tokens=2048,
                    max_seq_len=32768 + new)
    eng = aie.Engine(cfg, dtype="bf16", random_weights=True, seed=0, block_size=PAGE, **opts)
    prompts = [torch.randint(0, cfg["vocab_size"], (l,), generator=g).tolist() for l in lens]
    sp = aie.SamplingParams(max_tokens=new, ignore_eos=True)
    # warm-up: a prompt of more than one full portion and a few tokens (kernels and library products of both step sizes)
    warm = torch.randint(0, cfg["vocab_size"], (2048 + 100,), generator=g).tolist()
    eng.generate([warm], aie.SamplingParams(max_tokens=4, ignore_eos=True))
    torch.cuda.synchronize()
    model, kv_tok = eng.model, eng.cache.kv_bytes_per_token()
    wbytes = model.step_weight_bytes()
    stream = torch.cuda.current_stream()
    phases = {k: dict(steps=0, s=0.0, tokens=0, requests=0, max_tokens=0, bytes=0.0, flops=0.0, graph=0, host_bound=0)
              for k in ("decode", "prompt")}
    rids = [eng.add_request(p, sp) for p in prompts]
    generated = 0
    g0 = eng.runner.graph_launches
    marks = [torch.cuda.Event(enable_timing=True)]
    marks[0].record()
    owners = []
    t0 = time.perf_counter()
    while eng.has_unfinished() or eng._inflight:
        idle = stream.query()              # nothing left on the device before this step is launched: it waited for the host
        steps_before, gl = eng.counters["steps"], eng.runner.graph_launches
        generated += sum(1 for _, tok, _ in eng.step() if tok is not None)
        if eng.counters["steps"] == steps_before:
            continue
        ev = torch.cuda.Event(enable_timing=True)
        ev.record()
        marks.append(ev)
        ctx = eng.runner.last_ctx
        R, T = ctx.real_R, ctx.real_T
        ph = phases["decode" if T == R else "prompt"]
        owners.append(ph)
        held = float((ctx.h_ctx_len[:R] + ctx.h_q_len[:R]).sum())
        keys = float((ctx.h_q_len[:R] * ctx.h_ctx_len[:R] + ctx.h_q_len[:R] * (ctx.h_q_len[:R] + 1) / 2.0).sum()) / T
        ph["steps"] += 1
        ph["tokens"] += T
        ph["requests"] += R
        ph["max_tokens"] = max(ph["max_tokens"], T)
        ph["bytes"] += wbytes + kv_tok * held
        ph["flops"] += model.step_flops(T, keys, logit_rows=ctx.num_logit_rows)
        ph["graph"] += int(eng.runner.graph_launches > gl)
        ph["host_bound"] += int(bool(idle) and ph["steps"] > 1)
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    for i, ph in enumerate(owners):
        ph["s"] += marks[i].elapsed_time(marks[i + 1]) * 1e-3
    outs = [eng.take(r) for r in rids]
    st = eng.stats()
    assert all(len(o) == new for o in outs) and generated == n * new
    out = {"workload": name, "requests": n, "prompt_tokens": sum(lens), "generated_tokens": n * new,
           "seconds": round(dt, 3), "generated_tok_s": round(n * new / dt, 1),
           "total_tok_s": round((sum(lens) + n * new) / dt, 1), "steps": st["steps"], "preemptions": st["preemptions"],
           "peaks": pk["source"]}
    for k, ph in phases.items():
        if not ph["steps"]:
            continue
        sec = max(ph["s"], 1e-9)
        out[k] = {"steps": ph["steps"], "seconds": round(sec, 4), "tokens_per_s": round(ph["tokens"] / sec, 1),
                  "mean_tokens": round(ph["tokens"] / ph["steps"], 1), "max_tokens": ph["max_tokens"],
                  "mean_requests": round(ph["requests"] / ph["steps"], 1),
                  "gb_per_step": round(ph["bytes"] / ph["steps"] / 1e9, 3),
                  "hbm_gb_s": round(ph["bytes"] / sec / 1e9, 1), "hbm_frac": round(ph["bytes"] / sec / 1e9 / pk["hbm_gbs"], 4),
                  "tflop_s": round(ph["flops"] / sec / 1e12, 1),
                  "bf16_frac": round(ph["flops"] / sec / 1e12 / pk["bf16_tflops"], 4),
                  "graph_replayed_share": round(ph["graph"] / ph["steps"], 3),
                  "host_bound_share": round(ph["host_bound"] / ph["steps"], 3)}
    del eng
    torch.cuda.empty_cache()
    return out


def run_profile(torch, aie, model, batch, pk, prompt_len=PROMPT_LEN, context=CONTEXT):
    """CUDA-event time per class of kernel, launched eagerly: one 2,048-token prefill step, then 8 decode steps
    of `batch` requests with `prompt_len` cached tokens each.  Bytes and flops are what each launch has to move
    and do; frac is the larger of the two against the measured peaks, over the time."""
    from ai_engine_b200.cache import PagedCache
    from ai_engine_b200.engine.step import StepEntry, StepRunner
    from ai_engine_b200.kernels import profile
    from ai_engine_b200.sampling.sampler import Sampler

    g = torch.Generator().manual_seed(3)
    vocab = model.spec.vocab_size
    PROMPT_LEN, CONTEXT = prompt_len, max(context, prompt_len + 64)
    pages = (batch * (PROMPT_LEN + 32 + PAGE) + PREFILL_TOKENS) // PAGE + 8
    cache = PagedCache(model.cache_requests(), PAGE, pages, batch + 1, CONTEXT, model.dtype, model.device)
    runner = StepRunner(model, cache, use_graphs=False)
    sampler = Sampler(model.device)
    greedy = [aie.SamplingParams(max_tokens=1)] * batch
    slots = [cache.admit() for _ in range(batch + 1)]
    for s in slots[:batch]:
        cache.ensure(s, PROMPT_LEN + 32)
        ids = torch.randint(0, vocab, (PROMPT_LEN,), generator=g).tolist()
        for a in range(0, PROMPT_LEN, 2048):
            runner.step([StepEntry(s, a, ids[a:a + 2048], [])])
    cache.ensure(slots[batch], PREFILL_TOKENS)
    ids = torch.randint(0, vocab, (PREFILL_TOKENS,), generator=g).tolist()
    runner.step([StepEntry(slots[batch], 0, ids, [PREFILL_TOKENS - 1])])          # warm-up of the large step
    out = {}
    profile.start()
    runner.step([StepEntry(slots[batch], 0, ids, [PREFILL_TOKENS - 1])])
    out["prefill_2048"] = profile.stop(pk["hbm_gbs"], pk["bf16_tflops"])
    toks = torch.randint(0, vocab, (batch,), generator=g).tolist()
    step = lambda i: sampler.sample(runner.step([StepEntry(s, PROMPT_LEN + i, [toks[j]], [0])
                                                 for j, s in enumerate(slots[:batch])]), greedy, [0] * batch)
    for i in range(3):
        step(i)
    profile.start()
    for i in range(3, 11):
        step(i)
    rows = profile.stop(pk["hbm_gbs"], pk["bf16_tflops"])
    for r in rows:          # per step
        for k in ("calls", "ms", "gb", "gflop"):
            r[k] = round(r[k] / 8, 4)
    out[f"decode_b{batch}_per_step"] = rows
    runner.check_errors()
    return out


def config_record(layers, batch, peaks_source):
    """Every size of the run, flat (what is deeper than one level is lost in the record)."""
    c = LLAMA3_8B
    return {"model": "Llama-3-8B shape", "layers": layers, "layers_of_config": c["num_hidden_layers"],
            "hidden": c["hidden_size"], "heads": c["num_attention_heads"], "kv_heads": c["num_key_value_heads"],
            "head_dim": c["head_dim"], "intermediate": c["intermediate_size"], "vocab": c["vocab_size"],
            "global_batch": batch, "seq_len": PROMPT_LEN, "context": CONTEXT, "kv_page": PAGE,
            "parallelism": "single GPU", "l2": "inputs larger than L2 (weights read every step)",
            "peaks": peaks_source}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours")
    ap.add_argument("--layers", type=int, default=LLAMA3_8B["num_hidden_layers"],
                    help="run fewer layers than the configuration has (both numbers are reported)")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--skip-points", action="store_true")
    ap.add_argument("--workload", choices=["serving1b", "long3b"], default=None,
                    help="run one of the serving workloads through Engine.generate() and print its numbers")
    ap.add_argument("--only", choices=["decode", "prefill", "gemm", "attention", "peaks"], default=None,
                    help="time one part only and print its numbers (for profiling)")
    ap.add_argument("--profile", action="store_true",
                    help="CUDA-event time, bytes, flops and roofline fraction per class of kernel (eager launches)")
    ap.add_argument("--shape", choices=["8b", "1b", "3b"], default="8b",
                    help="layer sizes for --profile and --only decode|prefill (the headline run is always the 8B shape)")
    ap.add_argument("--prompt-len", type=int, default=PROMPT_LEN, help="cached tokens per request for --profile / --only decode")
    ap.add_argument("--skip-workloads", action="store_true", help="leave the 1B and 3B serving workloads out of `points`")
    a = ap.parse_args()
    if a.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "einyx/ai-engine is a Rust workspace (cargo/rustc are not installed, pip cannot "
                          "install it); no offline install of the reference is possible here"}))
        return 0
    if a.gpus != 1:
        print("bench.py: this engine runs on one GPU; --gpus %d is not supported" % a.gpus)
        return 2
    import torch

    import ai_engine_b200 as aie
    from ai_engine_b200.engine.loading import random_model

    warmup = max(a.warmup, 3)
    pk = peaks()
    if a.workload:
        print(json.dumps(run_workload(torch, aie, a.workload, pk)))
        return 0
    if a.only == "gemm":
        for k, v in time_gemms(torch, a.batch).items():
            print(k, json.dumps(v))
        return 0
    if a.only == "peaks":
        with ClockSampler() as clocks:
            r = time_peaks(torch)
        r["clocks"] = clocks.summary()
        print(json.dumps({"only": "peaks", **r}))
        return 0
    if a.only == "attention":
        for tokens, context in ((PREFILL_TOKENS, 0), (PREFILL_TOKENS, 6144), (512, 0), (200, 1000)):
            for k, v in time_attention(torch, tokens, context).items():
                print(k, json.dumps(v))
        g = torch.Generator().manual_seed(0)
        mixed = torch.randint(128, 4353, (64,), generator=g).tolist()
        for H, K, d, lens in ((32, 8, 128, [1024] * 8), (32, 8, 128, [1024] * 64), (32, 8, 128, [8192] * 8), (32, 8, 128, [1024]),
                              (32, 8, 64, [2600] * 56), (32, 8, 64, mixed), (24, 8, 128, [32768])):
            for k, v in time_decode_attention(torch, H, K, d, lens).items():
                print(k, json.dumps(v))
        return 0
    cfg = dict({"8b": LLAMA3_8B, "1b": LLAMA32_1B, "3b": LLAMA32_3B}[a.shape] if (a.profile or a.only) else LLAMA3_8B)
    if a.layers != LLAMA3_8B["num_hidden_layers"] or a.shape == "8b":
        cfg["num_hidden_layers"] = a.layers
    layers = cfg["num_hidden_layers"]
    model, _ = random_model(cfg, seed=0, dtype="bf16")
    if a.profile:
        from ai_engine_b200.kernels import profile
        for what, rows in run_profile(torch, aie, model, a.batch, pk, a.prompt_len).items():
            print(json.dumps({"profile": what, "shape": a.shape, "layers": layers, "prompt_len": a.prompt_len,
                              "peaks": pk["source"], "rows": rows}))
            print(f"-- {what} ({a.shape} shape, {layers} layers, {a.prompt_len} cached tokens a request)\n"
                  + profile.table(rows), file=sys.stderr)
        return 0
    if a.only:
        ctx_cap = max(CONTEXT, a.prompt_len + warmup + 5 * a.steps + 64)
        r = (time_decode(torch, aie, model, a.batch, a.prompt_len, a.steps, warmup, ctx_cap) if a.only == "decode"
             else time_prefill(torch, model, PREFILL_TOKENS, pk))
        if a.only == "decode":
            r["hbm_frac"] = r["bytes"] / (r["ms"] * 1e-3) / 1e9 / pk["hbm_gbs"]
        print(json.dumps({"only": a.only, "shape": a.shape, "layers": layers, "batch": a.batch, "prompt_len": a.prompt_len,
                          **{k: round(v, 4) for k, v in r.items()}}))
        return 0
    with ClockSampler() as clocks:
        main_pt = time_decode(torch, aie, model, a.batch, PROMPT_LEN, a.steps, warmup, CONTEXT)
    points = {}
    prefill = time_prefill(torch, model, PREFILL_TOKENS, pk)
    if not a.skip_points:
        for b in (1, 64):
            pt = time_decode(torch, aie, model, b, PROMPT_LEN, min(a.steps, 32), 3, CONTEXT, blocks=3)
            points[f"decode_b{b}"] = round(pt["tok_s"], 1)
            points[f"decode_b{b}_hbm_frac"] = round(pt["bytes"] / (pt["ms"] * 1e-3) / 1e9 / pk["hbm_gbs"], 4)
        long = time_decode(torch, aie, model, a.batch, CONTEXT - 128, min(a.steps, 32), 3, CONTEXT, blocks=3)
        points[f"decode_b{a.batch}_ctx{CONTEXT}"] = round(long["tok_s"], 1)
        points[f"decode_b{a.batch}_ctx{CONTEXT}_hbm_frac"] = round(long["bytes"] / (long["ms"] * 1e-3) / 1e9 / pk["hbm_gbs"], 4)
    del model
    torch.cuda.empty_cache()
    e2e, eng = time_e2e(torch, aie, cfg, a.batch, PROMPT_LEN, a.steps, warmup, a.layers)
    del eng
    torch.cuda.empty_cache()
    if not a.skip_points and not a.skip_workloads and a.layers == LLAMA3_8B["num_hidden_layers"]:
        w1 = run_workload(torch, aie, "serving1b", pk)
        points["serving1b_total_tok_s"] = w1["total_tok_s"]
        points["serving1b_decode_hbm_frac"] = w1.get("decode", {}).get("hbm_frac")
        points["serving1b_prompt_bf16_frac"] = w1.get("prompt", {}).get("bf16_frac")
        w3 = run_workload(torch, aie, "long3b", pk)
        points["long3b_prompt_tok_s"] = w3.get("prompt", {}).get("tokens_per_s")
        points["long3b_prompt_bf16_frac"] = w3.get("prompt", {}).get("bf16_frac")
        points["long3b_decode_tok_s"] = w3.get("decode", {}).get("tokens_per_s")
        points["long3b_decode_hbm_frac"] = w3.get("decode", {}).get("hbm_frac")
    achieved = main_pt["bytes"] / (main_pt["ms"] * 1e-3) / 1e9
    line = {
        "metric": "decode tok/s at batch 8 (Llama-3-8B shape, bf16, 1,024-token prompts, context 8,192)",
        "value": round(main_pt["tok_s"], 1), "unit": "tokens/s", "n_gpus": 1, "steps": a.steps,
        "warmup": warmup, "ms_per_step": round(main_pt["ms"], 4),
        "spread": {"blocks": main_pt["blocks"], "ms_min": round(main_pt["ms_min"], 4), "ms_max": round(main_pt["ms_max"], 4)},
        "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic: random weights N(0, 0.02), uniform random token ids",
        "impl": "ours",
        "config": config_record(a.layers, a.batch, pk["source"]),
        "e2e": {k: (round(v, 1) if isinstance(v, float) else v) for k, v in e2e.items()},
        "gpu_launches": main_pt["launches"],
        "prefill": {"value": round(prefill["value"], 1), "tokens": prefill["tokens"],
                    "ms": round(prefill["ms"], 3), "frac": round(prefill["frac"], 4),
                    "ms_min": round(prefill["ms_min"], 3), "ms_max": round(prefill["ms_max"], 3)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4)},
        "points": points,
        "clocks": clocks.summary(),
    }
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
