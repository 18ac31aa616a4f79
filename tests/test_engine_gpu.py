"""The engine through its Python entry point: greedy generation against the plain
implementation, batched == solo (the reference's batched_matches_solo,
crates/ai-engine-candle/tests/paged_batching.rs:41-51), preemption that reproduces the
same tokens, seeded temperature sampling, long decoding, and the command line."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_llama as pl
from helpers import FIXTURE_PROMPT, TINY, TOL_BF16, TOL_F32, make_fixture_dir, make_model_dir, plain_logits, random_ids

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def engine(d, name, dtype="fp32", **kw):
    import ai_engine_b200 as aie

    opts = dict(dtype=dtype, block_size=TINY[name][1]["block_size"], kv_cache_blocks=64,
                max_num_seqs=4, max_num_batched_tokens=64)
    opts.update(kw)
    return aie.Engine(d, **opts)


def greedy_with_margin(d, prompt, n, dtype, tol):
    """Greedy tokens from the plain implementation, and for each the gap between the
    best and second-best logit: a token is only compared where the gap exceeds what
    rounding could flip."""
    w, cfg = pl.read_weights(d, dtype), pl.read_config(d)
    ids, out, margins = list(prompt), [], []
    for _ in range(n):
        logits = pl.forward(w, cfg, ids)[-1]
        top = torch.topk(logits, 2).values
        t = int(torch.argmax(logits))
        out.append(t)
        margins.append(float(top[0] - top[1]))
        ids.append(t)
    return out, margins


def assert_differ_only_at_a_close_call(d, prompt, a, b, tol, what=""):
    """Two runs of one request (other batches, other portions) may part ways in bfloat16 only where the plain
    implementation, given what both agree on, has the two tokens within what rounding can flip."""
    if a == b:
        return
    i = next((k for k, (x, y) in enumerate(zip(a, b)) if x != y), None)
    assert i is not None, f"{what}: one run is a prefix of the other: {len(a)} and {len(b)} tokens"
    w, cfg = pl.read_weights(d, torch.float32), pl.read_config(d)
    logits = pl.forward(w, cfg, list(prompt) + list(a[:i]))[-1]
    gap = abs(float(logits[a[i]] - logits[b[i]]))
    top = float(logits.max())
    assert gap <= 2 * tol and top - float(min(logits[a[i]], logits[b[i]])) <= 2 * tol, \
        f"{what}: token {i}: {a[i]} against {b[i]}, logits {float(logits[a[i]])}, {float(logits[b[i]])}, best {top}"


def assert_same_until_a_close_call(got, want, margins, tol):
    for i, (g, w) in enumerate(zip(got, want)):
        if g != w:
            assert margins[i] <= 2 * tol, f"token {i}: got {g}, plain {w}, margin {margins[i]}"
            return                      # after a legitimate flip the sequences part ways
    assert len(got) == len(want)


@pytest.mark.parametrize("name,dtype", [("A", "fp32"), ("A", "bf16"), ("B", "fp32"), ("B", "bf16"), ("E", "bf16")])
def test_greedy_generation_matches_the_plain_implementation(tmp_path, name, dtype):
    import ai_engine_b200 as aie

    d = make_model_dir(tmp_path, name)
    vocab = TINY[name][0]["vocab_size"]
    lens = (5, 17, 33) if name == "A" else ((1, 9, 40, 120) if name == "B" else (3, 150, 300, 64))
    prompts = [random_ids(n, vocab, 30 + n) for n in lens]
    eng = engine(d, name, dtype, max_num_batched_tokens=16 if name == "B" else (200 if name == "E" else 64))
    outs = eng.generate(prompts, aie.SamplingParams(max_tokens=8, ignore_eos=True))
    tol = TOL_F32 if dtype == "fp32" else TOL_BF16
    for p, o in zip(prompts, outs):
        want, margins = greedy_with_margin(d, p, 8, torch.float64 if dtype == "fp32" else torch.float32, tol)
        assert_same_until_a_close_call(o, want, margins, tol)
    st = eng.stats()
    assert st["finished"] == len(prompts) and st["cache"]["group0"]["in_use"] == 0


@pytest.mark.parametrize("dtype", ["fp32", "bf16"])
def test_generation_from_the_references_fixture(tmp_path, dtype):
    """Engine.generate() on the reference's golden fixture: the first token after its prompt is the argmax of
    the reference's logits (150), and the continuation is the plain implementation's."""
    import ai_engine_b200 as aie

    d = make_fixture_dir(tmp_path, "float32" if dtype == "fp32" else "bfloat16")
    eng = engine(d, "Q", dtype)
    prompts = [FIXTURE_PROMPT, random_ids(30, 512, 8)]
    outs = eng.generate(prompts, aie.SamplingParams(max_tokens=10, ignore_eos=True))
    assert outs[0][0] == 150
    tol = TOL_F32 if dtype == "fp32" else TOL_BF16
    for p, o in zip(prompts, outs):
        want, margins = greedy_with_margin(d, p, 10, torch.float64 if dtype == "fp32" else torch.float32, tol)
        assert_same_until_a_close_call(o, want, margins, tol)


@pytest.mark.parametrize("dtype", ["fp32", "bf16"])
def test_batched_matches_solo(tmp_path, dtype):
    import ai_engine_b200 as aie

    d = make_model_dir(tmp_path, "B")
    prompts = [random_ids(n, 384, 50 + n) for n in (3, 21, 8, 64)]
    sp = aie.SamplingParams(max_tokens=24, ignore_eos=True)
    solo = [engine(d, "B", dtype, max_num_seqs=1).generate([p], sp)[0] for p in prompts]
    together = engine(d, "B", dtype, max_num_seqs=4, max_num_batched_tokens=16).generate(prompts, sp)
    if dtype == "fp32":
        assert together == solo            # float32: the same bits whatever the batch
    else:                                  # bfloat16: another batch size may round a near-tie the other way
        for p, a, b in zip(prompts, together, solo):
            assert_differ_only_at_a_close_call(d, p, a, b, TOL_BF16, f"prompt of {len(p)}")


def test_preemption_reproduces_the_same_tokens(tmp_path):
    import ai_engine_b200 as aie

    d = make_model_dir(tmp_path, "A")
    prompts = [random_ids(n, 256, 70 + n) for n in (20, 25, 30)]
    params = [aie.SamplingParams(max_tokens=30, ignore_eos=True),
              aie.SamplingParams(max_tokens=30, ignore_eos=True, temperature=0.8, seed=7),
              aie.SamplingParams(max_tokens=30, ignore_eos=True, temperature=1.1, seed=8, top_k=40)]
    roomy = engine(d, "A", "fp32", kv_cache_blocks=64).generate(prompts, params)
    tight_engine = engine(d, "A", "fp32", kv_cache_blocks=9)       # 144 tokens for 3 x 50..60
    tight = tight_engine.generate(prompts, params)
    assert tight_engine.stats()["preemptions"] >= 1
    assert tight == roomy


def test_seeded_sampling_is_reproducible_and_seed_matters(tmp_path):
    import ai_engine_b200 as aie

    d = make_model_dir(tmp_path, "B")
    prompts = [random_ids(n, 384, 90 + n) for n in (1, 9, 40, 120)]
    sp = lambda s: aie.SamplingParams(max_tokens=12, temperature=0.8, seed=s, ignore_eos=True)
    a = engine(d, "B", "fp32", max_num_batched_tokens=16).generate(prompts, sp(3))
    b = engine(d, "B", "fp32", max_num_batched_tokens=16).generate(prompts, sp(3))
    c = engine(d, "B", "fp32", max_num_batched_tokens=16).generate(prompts, sp(4))
    assert a == b and a != c
    # the first sampled token of each request against the plain sampler on plain logits
    from ai_engine_b200.sampling.rng import uniform
    for p, o in zip(prompts, a):
        logits = plain_logits(d, p)[-1]
        want = pl.sample(logits.tolist(), 0.8, r=uniform(3, 0))
        near = {pl.sample(logits.tolist(), 0.8, r=min(max(uniform(3, 0) + dr, 0.0), 1.0)) for dr in (-1e-4, 1e-4)}
        assert o[0] == want or o[0] in near


def test_eos_ends_a_request_and_is_not_returned(tmp_path):
    import ai_engine_b200 as aie

    d = make_model_dir(tmp_path, "A")
    p = random_ids(12, 256, 5)
    free = engine(d, "A", "fp32").generate([p], aie.SamplingParams(max_tokens=10, ignore_eos=True))[0]
    cfgp = os.path.join(d, "config.json")
    raw = json.load(open(cfgp))
    raw["eos_token_id"] = [free[4], 99999]
    json.dump(raw, open(cfgp, "w"))
    stopped = engine(d, "A", "fp32").generate([p], aie.SamplingParams(max_tokens=10))[0]
    assert stopped == free[:free.index(free[4])]


@pytest.mark.parametrize("dtype", ["fp32", "bf16"])
def test_running_a_step_ahead_changes_no_token(tmp_path, dtype):
    """The host launches step n + 1 before it has read step n's tokens (they are handed over on the
    device).  Same tokens as the loop that reads every token first: with requests that end by an EOS
    seen one step late, by length, with sampling, and with so few pages that requests are preempted."""
    import ai_engine_b200 as aie

    d = make_model_dir(tmp_path, "A")
    prompts = [random_ids(n, 256, 40 + n) for n in (3, 20, 25, 30, 7, 50)]
    free = engine(d, "A", dtype, async_scheduling=False).generate(
        prompts, aie.SamplingParams(max_tokens=24, ignore_eos=True))
    cfgp = os.path.join(d, "config.json")
    raw = json.load(open(cfgp))
    raw["eos_token_id"] = [free[0][5], free[2][11], free[3][0]]       # ends some requests early, one at its first token
    json.dump(raw, open(cfgp, "w"))
    params = [aie.SamplingParams(max_tokens=24), aie.SamplingParams(max_tokens=40, ignore_eos=True),
              aie.SamplingParams(max_tokens=24, temperature=0.9, seed=5), aie.SamplingParams(max_tokens=24),
              aie.SamplingParams(max_tokens=1),
              aie.SamplingParams(max_tokens=40, temperature=1.2, seed=6, top_p=0.9, ignore_eos=True)]
    outs = {}
    for ahead in (False, True):
        for blocks in (64, 8):
            eng = engine(d, "A", dtype, async_scheduling=ahead, kv_cache_blocks=blocks)
            outs[ahead, blocks] = eng.generate(prompts, params)
            st = eng.stats()
            assert st["running"] == 0 and st["waiting"] == 0 and not eng._inflight
            assert all(g["in_use"] == 0 for g in st["cache"].values()), st["cache"]
            if blocks == 8:
                assert st["preemptions"] >= 1
    eos = set(raw["eos_token_id"])
    assert all(not (set(o) & eos) for o, sp in zip(outs[True, 64], params) if not sp.ignore_eos)
    assert len(outs[True, 64][0]) <= 5 and outs[True, 64][3] == [] and len(outs[True, 64][4]) <= 1
    if dtype == "fp32":
        assert outs[True, 64] == outs[False, 64] == outs[True, 8] == outs[False, 8]
    else:       # bf16: a preempted request is recomputed in other portions, which may round a close call the other way
        assert outs[True, 64] == outs[False, 64] and outs[True, 8] == outs[False, 8]


@pytest.mark.parametrize("seed", [1, 2, 3])
def test_random_workloads_step_ahead_against_step_by_step(tmp_path, seed):
    """Random prompts, lengths, sampling options, EOS sets, token budgets and pool sizes (float32, where the
    two loops must agree token for token): the engine a step ahead of the device against the engine that reads
    every token first; all pages come back."""
    import ai_engine_b200 as aie

    rng = np.random.RandomState(seed)
    d = make_model_dir(tmp_path, "B")
    n = int(rng.randint(3, 9))
    prompts = [random_ids(int(rng.randint(1, 90)), 384, 1000 * seed + i) for i in range(n)]
    cfgp = os.path.join(d, "config.json")
    raw = json.load(open(cfgp))
    raw["eos_token_id"] = [int(t) for t in rng.randint(0, 384, size=40)]      # a tenth of the vocabulary ends a request
    json.dump(raw, open(cfgp, "w"))
    params = []
    for i in range(n):
        kind = rng.randint(0, 3)
        params.append(aie.SamplingParams(max_tokens=int(rng.randint(1, 40)), ignore_eos=bool(rng.randint(0, 4) == 0),
                                         temperature=[0.0, 0.7, 1.3][kind], seed=int(rng.randint(0, 1000)),
                                         top_k=[None, None, 20][int(rng.randint(0, 3))], top_p=[None, 0.9][int(rng.randint(0, 2))]))
    page = TINY["B"][1]["block_size"]
    need = max((len(p) + sp.max_tokens + page - 1) // page for p, sp in zip(prompts, params))
    opts = dict(kv_cache_blocks=int(need + rng.randint(0, 6)), max_num_batched_tokens=int(rng.choice([16, 32, 64])),
                max_num_seqs=int(rng.randint(2, 5)))
    outs = []
    for ahead in (False, True):
        eng = engine(d, "B", "fp32", async_scheduling=ahead, **opts)
        outs.append(eng.generate(prompts, params))
        st = eng.stats()
        assert st["running"] == 0 and st["waiting"] == 0 and not eng._inflight
        assert all(g["in_use"] == 0 for g in st["cache"].values())
    assert outs[0] == outs[1]
    eos = set(raw["eos_token_id"])
    for o, sp in zip(outs[0], params):
        assert len(o) <= sp.max_tokens and (sp.ignore_eos or not (set(o) & eos))


def test_stepping_by_hand_and_taking_finished_requests(tmp_path):
    import ai_engine_b200 as aie

    d = make_model_dir(tmp_path, "A")
    eng = engine(d, "A", "fp32")
    want = engine(d, "A", "fp32").generate([random_ids(9, 256, 3), random_ids(30, 256, 4)],
                                             aie.SamplingParams(max_tokens=7, ignore_eos=True))
    a = eng.add_request(random_ids(9, 256, 3), aie.SamplingParams(max_tokens=7, ignore_eos=True))
    b = eng.add_request(random_ids(30, 256, 4), aie.SamplingParams(max_tokens=7, ignore_eos=True))
    with pytest.raises(KeyError):
        eng.take(a)
    streamed = {a: [], b: []}
    done = set()
    while eng.has_unfinished() or eng._inflight:
        for rid, tok, fin in eng.step():
            if tok is not None:
                streamed[rid].append(tok)
            if fin:
                done.add(rid)
    assert done == {a, b}
    assert [eng.take(a), eng.take(b)] == want == [streamed[a], streamed[b]]
    assert not eng.requests


def test_long_decoding_and_first_tokens(tmp_path):
    """300 tokens decoded one by one after a 3-token prompt: logits of the first tokens and
    of every decoded position against the plain implementation run on the final sequence."""
    from ai_engine_b200.engine.replay import Replayer

    d = make_model_dir(tmp_path, "C")
    ids = random_ids(303, 200, 17)
    ref = plain_logits(d, ids, torch.float64)
    rep = Replayer(d, "float32", max_tokens=320, block_size=16)
    got = [rep.run_step([dict(id="x", tokens=ids[:3], want=[0, 1, 2])]).numpy()]
    for t in ids[3:]:
        got.append(rep.run_step([dict(id="x", tokens=[t], want=[0])]).numpy())
    got = np.concatenate(got).astype(np.float64)
    err = np.abs(got - ref).max(axis=1)
    assert err.max() <= TOL_F32, f"first wrong token {int(np.argmax(err > TOL_F32))}"
    rep16 = Replayer(d, "bfloat16", max_tokens=320, block_size=16)
    ref32 = plain_logits(d, ids, torch.float32)
    g = [rep16.run_step([dict(id="x", tokens=ids[:3], want=[0, 1, 2])]).numpy()]
    for t in ids[3:]:
        g.append(rep16.run_step([dict(id="x", tokens=[t], want=[0])]).numpy())
    err = np.abs(np.concatenate(g) - ref32).max(axis=1)
    assert err.max() <= TOL_BF16, f"first wrong token {int(np.argmax(err > TOL_BF16))}"


def test_rejections_and_bad_options(tmp_path):
    import ai_engine_b200 as aie

    d = make_model_dir(tmp_path, "A")
    eng = engine(d, "A", "fp32", kv_cache_blocks=4, max_seq_len=128)
    with pytest.raises(ValueError, match="never fit"):
        eng.add_request(list(range(100)), aie.SamplingParams(max_tokens=5))
    with pytest.raises(ValueError, match="outside the vocabulary"):
        eng.add_request([1, 2, 999])
    with pytest.raises(ValueError, match="max context"):
        eng.add_request([1] * 200)
    with pytest.raises(ValueError, match="cuda:0 only"):
        aie.Engine(d, device="cpu")
    with pytest.raises(ValueError, match="unknown engine option"):
        aie.Engine(d, pool_sizes=3)


def test_command_line(tmp_path):
    d = make_model_dir(tmp_path, "A")
    cfg = tmp_path / "provider.toml"
    cfg.write_text(f'[[provider]]\nid = "local"\nkind = "b200"\nweights_path = "{d}"\n'
                   'device = "cuda:0"\ndtype = "fp32"\nmax_num_seqs = 2\nblock_size = 16\nkv_cache_blocks = 32\n')
    exe = [sys.executable, os.path.join(ROOT, "bin", "ai-engine")]
    assert subprocess.run(exe + ["-c", str(cfg), "--check"], capture_output=True, text=True).stdout.strip() == "ok"
    p = subprocess.run(exe + ["-c", str(cfg), "--prompt-ids", "5,17,3", "--prompt-ids", "9,9", "--max-tokens", "6",
                              "--ignore-eos", "--stats", "--profile"], capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-1500:]
    assert "kernel class" in p.stderr and "gemm_f32" in p.stderr and "attention_plain" in p.stderr
    lines = [[int(t) for t in l.split(",")] for l in p.stdout.strip().splitlines()]
    assert len(lines) == 2 and all(len(l) == 6 for l in lines)
    want, margins = greedy_with_margin(d, [5, 17, 3], 6, torch.float64, TOL_F32)
    assert_same_until_a_close_call(lines[0], want, margins, TOL_F32)
    bad = subprocess.run(exe + ["--model", str(tmp_path / "none"), "--prompt-ids", "1"], capture_output=True, text=True)
    assert bad.returncode == 1 and "error" in bad.stderr


def test_kernel_classes_are_timed_on_request(tmp_path):
    """Profiling on: every launch of a step sits between two CUDA events under its class's name, with the
    bytes and flops it has to move and do; off (the default): nothing is recorded."""
    from ai_engine_b200.engine.replay import Replayer
    from ai_engine_b200.kernels import profile

    d = make_model_dir(tmp_path, "E")
    rep = Replayer(d, "bfloat16", max_tokens=512, block_size=16)
    ids = random_ids(200, 260, 2)
    rep.run_step([dict(id="x", tokens=ids[:150], want=[149])])
    assert not profile.enabled() and not profile._RECORDS
    profile.start()
    rep.run_step([dict(id="y", tokens=ids[:150], want=[149])])
    rep.run_step([dict(id="y", tokens=ids[150:151], want=[0]), dict(id="x", tokens=ids[150:151], want=[0])])
    rows = {r["kernel"]: r for r in profile.stop(6500.0, 1600.0)}
    assert not profile.enabled()
    for cls in ("embed_gather", "add_rmsnorm", "gemm_library", "rope_kv_write", "attention_prefill_tcgen05", "silu_mul",
                "gemm_tc", "gemm_tc_rope", "gemm_tc_swiglu", "attention_decode"):
        assert cls in rows and rows[cls]["ms"] > 0 and rows[cls]["gb"] > 0, (cls, sorted(rows))
    L, D, F = 2, 256, 320
    assert rows["gemm_library"]["calls"] == 4 * L         # qkv, o, gate_up, down of the 150-token step (its one logits row: gemm_tc)
    assert abs(rows["gemm_library"]["gflop"] - 2 * 150 * L * (D * (4 + 4) * 128 + 4 * 128 * D + 3 * F * D) / 1e9) < 0.01
    assert abs(rows["attention_prefill_tcgen05"]["gflop"] - 4 * 128 * 4 * (150 * 151 / 2) * L / 1e9) < 0.01
    assert abs(rows["attention_decode"]["gb"] - 2 * 151 * 2 * 128 * 2 * 2 * L / 1e9) < 1e-4
    assert abs(sum(r["share"] for r in rows.values()) - 1.0) < 1e-2


def test_decode_steps_replayed_from_a_graph_match_eager_steps(tmp_path):
    """bfloat16 decode steps are captured once per layout and replayed; the logits must be
    the ones the same step gives when every kernel is launched afresh."""
    from ai_engine_b200.cache import PagedCache
    from ai_engine_b200.engine.loading import load_model
    from ai_engine_b200.engine.step import StepEntry, StepRunner

    d = make_model_dir(tmp_path, "D")
    model, _ = load_model(d, "bfloat16")
    ids = [random_ids(40 + 3 * i, 300, 60 + i) for i in range(3)]
    outs = {}
    for graphs in (False, True):
        cache = PagedCache(model.cache_requests(), 16, 64, 4, 2048, model.dtype, model.device)
        runner = StepRunner(model, cache, use_graphs=graphs)
        slots = [cache.admit() for _ in ids]
        for s, p in zip(slots, ids):
            cache.ensure(s, len(p) + 40)
            runner.step([StepEntry(s, 0, p[:20], [])])
        got = []
        for k in range(20):
            got.append(runner.step([StepEntry(s, 20 + k, [p[20 + k]], [0]) for s, p in zip(slots, ids)]).cpu())
        runner.check_errors()
        outs[graphs] = torch.stack(got)
        if graphs:
            assert runner.graphs_captured == 1 and runner.graph_launches > 0
    # the replayed step cuts the keys into as many parts as its layout's widest request could
    # need, the eager step into as many as this step needs: equal up to bfloat16 rounding
    assert (outs[True] - outs[False]).abs().max() <= 1e-2
    ref = plain_logits(d, ids[1][:40], torch.float32)
    assert np.abs(outs[True][:, 1].numpy() - ref[20:40]).max() <= TOL_BF16


def test_decode_batches_rounded_up_to_a_multiple_of_eight_share_a_graph(tmp_path):
    """Decode steps of 9 to 16 requests run as 16 rows (the entry with the shortest cache repeated): one layout, one graph, and
    the logits of every live row are what the step of exactly those rows gives, and the plain implementation's."""
    from ai_engine_b200.cache import PagedCache
    from ai_engine_b200.engine.loading import load_model
    from ai_engine_b200.engine.step import StepEntry, StepRunner

    d = make_model_dir(tmp_path, "D")
    model, _ = load_model(d, "bf16")
    page = TINY["D"][1]["block_size"]
    prompts = [random_ids(16 + s, 300, 200 + s) for s in range(13)]
    refs = [plain_logits(d, p, torch.float32) for p in prompts]
    lives = [13, 12, 11, 13, 10, 9]            # requests 0 .. live-1 bring their next token: all within one bucket of 16
    outs = {}
    for graphs in (False, True):
        cache = PagedCache(model.cache_requests(), page, 64, 16, 256, model.dtype, model.device)
        runner = StepRunner(model, cache, use_graphs=graphs)
        slots = [cache.admit() for _ in range(13)]
        at = [len(p) - 6 for p in prompts]
        for s, p, n in zip(slots, prompts, at):
            assert cache.ensure(s, len(p))
            runner.step([StepEntry(s, 0, p[:n], [])])
        got = []
        for live in lives:
            es = [StepEntry(slots[r], at[r], [prompts[r][at[r]]], [0]) for r in range(live)]
            lg = runner.step(es)
            assert lg.shape[0] == live
            lg = lg.float().cpu()
            for r in range(live):
                assert np.abs(lg[r].numpy() - refs[r][at[r]]).max() <= TOL_BF16, (graphs, live, r)
                at[r] += 1
            got.append(lg)
        runner.check_errors()
        outs[graphs] = got
        if graphs:
            assert runner.graphs_captured == 1 and runner.graph_launches > 0
    for a, b in zip(outs[True], outs[False]):
        assert (a - b).abs().max() <= 1e-2      # other split counts of the attention: rounding only


@pytest.mark.parametrize("name", ["D", "E"])
def test_the_bfloat16_engine_as_it_is_served(tmp_path, name):
    """What serving runs, against the plain implementation: the fast attention kernels (head size 64 and 128),
    captured graphs, more than eight live requests (decode batches wander through 9 .. 14 rows, rounded up by
    repeated rows, and below 8 as requests end by EOS or length), ids handed over on the device, a roomy
    pool and one so tight that requests are preempted, the host a step ahead of the device and not."""
    import ai_engine_b200 as aie

    d = make_model_dir(tmp_path, name)
    vocab = TINY[name][0]["vocab_size"]
    rng = np.random.RandomState(7)
    lens = [3, 150, 41, 9, 77, 20, 118, 5, 64, 33, 90, 12, 27, 55]
    prompts = [random_ids(n, vocab, 300 + i) for i, n in enumerate(lens)]
    news = [int(n) for n in rng.randint(8, 40, size=len(lens))]
    opts = dict(max_num_seqs=16, max_num_batched_tokens=96)
    free = engine(d, name, "bf16", kv_cache_blocks=256, **opts).generate(
        prompts, [aie.SamplingParams(max_tokens=n, ignore_eos=True) for n in news])
    cfgp = os.path.join(d, "config.json")
    raw = json.load(open(cfgp))
    raw["eos_token_id"] = sorted({free[1][6], free[4][7], free[8][2], free[11][0]})    # ends some requests mid-flight
    json.dump(raw, open(cfgp, "w"))
    eos = set(raw["eos_token_id"])
    params = [aie.SamplingParams(max_tokens=n, ignore_eos=(i % 5 == 0)) for i, n in enumerate(news)]
    page = TINY[name][1]["block_size"]
    need = sum((len(p) + n + page - 1) // page for p, n in zip(prompts, news))
    w, cfg = pl.read_weights(d, torch.float32), pl.read_config(d)
    outs = {}
    for blocks in (need + 8, need // 3):
        for ahead in (False, True):
            eng = engine(d, name, "bf16", kv_cache_blocks=blocks, async_scheduling=ahead, **opts)
            outs[blocks, ahead] = eng.generate(prompts, params)
            st = eng.stats()
            assert eng.runner.graphs_captured >= 1 and eng.runner.pad_decode
            assert st["running"] == 0 and st["waiting"] == 0 and not eng._inflight
            assert all(g["in_use"] == 0 for g in st["cache"].values()), st["cache"]
            assert (st["preemptions"] >= 1) == (blocks < need), (blocks, need, st["preemptions"])
        for p, a, b in zip(prompts, outs[blocks, True], outs[blocks, False]):
            assert_differ_only_at_a_close_call(d, p, a, b, TOL_BF16, f"pool {blocks}, a step ahead or not")
    for key, got in outs.items():
        for i, (p, sp, o) in enumerate(zip(prompts, params, got)):
            want, margins = greedy_with_margin(d, p, sp.max_tokens, torch.float32, TOL_BF16)
            parted = False
            for k, (g, x) in enumerate(zip(o, want)):
                if g != x:
                    assert margins[k] <= 2 * TOL_BF16, f"{key} request {i} token {k}: got {g}, plain {x}, margin {margins[k]}"
                    parted = True
                    break
            if parted:
                continue
            assert sp.ignore_eos or not (set(o) & eos), (key, i)
            if len(o) < sp.max_tokens:            # it ended early: the plain continuation's next token is an EOS
                assert not sp.ignore_eos and (want[len(o)] in eos or margins[len(o)] <= 2 * TOL_BF16), (key, i, len(o))
