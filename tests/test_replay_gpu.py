"""Trace replay on the GPU against the plain implementation: each request alone
and whole; most of it in one step and the last 32 tokens one by one; portions of
changing size down to two tokens; and up to four live requests mixed, portions
of some beside decoded tokens of others, with so few pages that they are used
again.  In float32 and in bfloat16, at the tiny configurations."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

from helpers import (TINY, TOL_BF16, TOL_F32, TOL_F32_SCHEDULES, make_model_dir, plain_logits,
                     random_ids)

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def tol_for(dtype):
    return TOL_F32 if dtype == "float32" else TOL_BF16


def oracle_dtype(dtype):
    return torch.float64 if dtype == "float32" else torch.float32


def replayer(model_dir, dtype, name, max_tokens, max_num_seqs=4):
    from ai_engine_b200.engine.replay import Replayer

    return Replayer(model_dir, dtype, max_tokens=max_tokens, block_size=TINY[name][1]["block_size"],
                    max_num_seqs=max_num_seqs)


def whole(rep, rid, ids):
    out = rep.run_step([dict(id=rid, tokens=ids, want=list(range(len(ids))))], end=[rid])
    return out.numpy().astype(np.float64)


CASES = [("A", "float32"), ("A", "bfloat16"), ("B", "float32"), ("B", "bfloat16"),
         ("D", "float32"), ("D", "bfloat16"), ("E", "bfloat16")]


@pytest.mark.parametrize("name,dtype", CASES)
def test_whole_prompts(tmp_path, name, dtype):
    d = make_model_dir(tmp_path, name)
    vocab = TINY[name][0]["vocab_size"]
    rep = replayer(d, dtype, name, max_tokens=128)
    for n, seed in ((1, 3), (5, 4), (17, 5), (33, 6), (120, 7)):
        ids = random_ids(n, vocab, seed)
        got = whole(rep, f"r{n}", ids)
        ref = plain_logits(d, ids, oracle_dtype(dtype))
        assert got.shape == ref.shape
        assert np.abs(got - ref).max() <= tol_for(dtype), (n, np.abs(got - ref).max())
    rep.cache.book.check_invariants()
    assert rep.cache.book.pages_in_use(0) == 0


@pytest.mark.parametrize("name,dtype", CASES)
def test_last_32_one_by_one(tmp_path, name, dtype):
    d = make_model_dir(tmp_path, name)
    vocab = TINY[name][0]["vocab_size"]
    ids = random_ids(100, vocab, 11)
    ref = plain_logits(d, ids, oracle_dtype(dtype))
    rep = replayer(d, dtype, name, max_tokens=128)
    got = [rep.run_step([dict(id="x", tokens=ids[:68], want=list(range(68)))]).numpy()]
    for i in range(68, 100):
        got.append(rep.run_step([dict(id="x", tokens=[ids[i]], want=[0])]).numpy())
    rep.run_step([], end=["x"])
    got = np.concatenate(got).astype(np.float64)
    err = np.abs(got - ref).max(axis=1)
    assert err.max() <= tol_for(dtype), f"first wrong token {int(np.argmax(err > tol_for(dtype)))}: {err.max()}"
    if dtype == "float32":
        rep2 = replayer(d, dtype, name, max_tokens=128)
        assert np.abs(whole(rep2, "w", ids) - got).max() <= TOL_F32_SCHEDULES


PORTIONS = [2, 3, 7, 16, 5, 2, 13, 2, 31, 9, 2, 8]   # sums to 100


@pytest.mark.parametrize("name,dtype", CASES)
def test_portions_of_changing_size(tmp_path, name, dtype):
    d = make_model_dir(tmp_path, name)
    vocab = TINY[name][0]["vocab_size"]
    ids = random_ids(sum(PORTIONS), vocab, 12)
    ref = plain_logits(d, ids, oracle_dtype(dtype))
    rep = replayer(d, dtype, name, max_tokens=128)
    got, at = [], 0
    for p in PORTIONS:
        got.append(rep.run_step([dict(id="x", tokens=ids[at:at + p], want=list(range(p)))]).numpy())
        at += p
    got = np.concatenate(got).astype(np.float64)
    err = np.abs(got - ref).max(axis=1)
    assert err.max() <= tol_for(dtype), f"first wrong token {int(np.argmax(err > tol_for(dtype)))}: {err.max()}"


def mixed_trace(lengths, vocab, seed):
    """Up to four live requests; each is fed in portions of changing size and then
    token by token while others are mid-prompt; finished requests leave and new
    ones take their pages.  Returns (steps, {id: ids})."""
    rng = np.random.RandomState(seed)
    seqs = {f"q{i}": random_ids(n, vocab, seed + 10 + i) for i, n in enumerate(lengths)}
    pending = list(seqs)
    live, fed, steps = [], {}, []
    while pending or live:
        while pending and len(live) < 4:
            rid = pending.pop(0)
            live.append(rid)
            fed[rid] = 0
        entries, end = [], []
        for rid in list(live):
            if rng.rand() < 0.2 and len(live) > 1:
                continue                      # left out of this step, goes on later
            left = len(seqs[rid]) - fed[rid]
            decode_phase = left <= 12
            n = 1 if decode_phase else int(min(left - 12, rng.choice([2, 3, 5, 8, 16, 21])))
            if not decode_phase and left - 12 - n == 1:
                n += 1
            toks = seqs[rid][fed[rid]:fed[rid] + n]
            entries.append(dict(id=rid, tokens=toks, want=list(range(n)), at=fed[rid]))
            fed[rid] += n
            if fed[rid] == len(seqs[rid]):
                end.append(rid)
                live.remove(rid)
        if entries:
            steps.append(dict(step=len(steps), entries=entries, end=end))
    return steps, seqs


def pool_tokens_for(steps, seqs):
    """The most tokens live requests hold at any time, each rounded up to 64."""
    held, peak = {}, 0
    for s in steps:
        for e in s["entries"]:
            held[e["id"]] = e["at"] + len(e["tokens"])
        peak = max(peak, sum((v + 63) // 64 * 64 for v in held.values()))
        for rid in s["end"]:
            held.pop(rid)
    return peak


@pytest.mark.parametrize("name,dtype", CASES)
def test_mixed_requests_with_pages_used_again(tmp_path, name, dtype):
    d = make_model_dir(tmp_path, name)
    vocab = TINY[name][0]["vocab_size"]
    lengths = [40, 9, 120, 1, 77, 33, 64, 18, 100]
    steps, seqs = mixed_trace(lengths, vocab, 21)
    rep = replayer(d, dtype, name, max_tokens=pool_tokens_for(steps, seqs))
    refs = {rid: plain_logits(d, ids, oracle_dtype(dtype)) for rid, ids in seqs.items()}
    worst = 0.0
    for s in steps:
        out = rep.run_step(s["entries"], s["end"]).numpy().astype(np.float64)
        row = 0
        for e in s["entries"]:
            n = len(e["tokens"])
            ref = refs[e["id"]][e["at"]:e["at"] + n]
            err = np.abs(out[row:row + n] - ref).max()
            assert err <= tol_for(dtype), f"step {s['step']} request {e['id']} at {e['at']}: {err}"
            worst = max(worst, err)
            row += n
        rep.cache.book.check_invariants()
    # the pool was too small to serve every request from fresh pages
    total_pages = rep.cache.book.group(0).num_pages
    assert rep.cache.book.total_allocations(0) > total_pages
    assert rep.cache.book.pages_in_use(0) == 0


def test_trace_run_program(tmp_path):
    """bin/trace_run as a user starts it: JSON lines in, <step>.f32 out, `done <step>`."""
    d = make_model_dir(tmp_path, "A")
    ids = random_ids(40, 256, 5)
    out_dir = os.path.join(str(tmp_path), "out")
    lines = [dict(step=0, entries=[dict(id="a", tokens=ids[:30], want=[0, 29])], end=[]),
             dict(step=1, entries=[dict(id="a", tokens=ids[30:32], want=[])], end=[]),
             dict(step=2, entries=[dict(id="a", tokens=ids[32:], want=[7]),
                                   dict(id="b", tokens=ids[:3], want=[2])], end=["a", "b"])]
    p = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", d,
                        "--dtype", "float32", "--out", out_dir, "--max-tokens", "128"],
                       input="\n".join(json.dumps(l) for l in lines) + "\n", text=True,
                       capture_output=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    assert p.stdout.split() == ["done", "0", "done", "1", "done", "2"]
    ref = plain_logits(d, ids)
    s0 = np.fromfile(os.path.join(out_dir, "0.f32"), dtype="<f4").reshape(2, 256)
    s2 = np.fromfile(os.path.join(out_dir, "2.f32"), dtype="<f4").reshape(2, 256)
    assert not os.path.exists(os.path.join(out_dir, "1.f32"))
    assert np.abs(s0 - ref[[0, 29]]).max() <= TOL_F32
    assert np.abs(s2[0] - ref[39]).max() <= TOL_F32
    assert np.abs(s2[1] - ref[2]).max() <= TOL_F32
