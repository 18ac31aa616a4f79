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

from helpers import (FIXTURE_PROMPT, TINY, TOL_BF16, TOL_F32, TOL_F32_SCHEDULES, fixture_reference_logits,
                     make_fixture_dir, make_model_dir, plain_logits, random_ids)

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
         ("D", "float32"), ("D", "bfloat16"), ("E", "bfloat16"), ("Q", "float32"), ("Q", "bfloat16")]


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


@pytest.mark.parametrize("name", ["D", "E"])
def test_cached_keys_do_not_depend_on_how_the_prompt_was_cut(tmp_path, name):
    """bfloat16: the keys and values a prompt leaves in its pages, fed whole (one step of 150 tokens: library
    products) and in portions (steps of 40, 64, 30, 13 and 3 tokens: this package's products, the last with the
    rotation in the product's epilogue).  The projection reaches the rotation in float32 either way and is
    rounded once, so the pages agree to the last bit almost everywhere, and nowhere differ by more than one
    step of bfloat16 (products that sum in another order may land on the other side of a rounding boundary)."""
    d = make_model_dir(tmp_path, name)
    ids = random_ids(150, TINY[name][0]["vocab_size"], 44)
    pools = []
    for portions in ([150], [40, 64, 30, 13, 3]):
        rep = replayer(d, "bfloat16", name, max_tokens=192)
        at = 0
        for n in portions:
            rep.run_step([dict(id="x", tokens=ids[at:at + n], want=[])])
            at += n
        pages = (150 + 15) // 16
        pool = rep.cache.groups[0].pool[:, :, :pages].float().cpu()       # [runs, k|v, pages, K, page, d]
        pools.append(pool.permute(0, 1, 2, 4, 3, 5).reshape(pool.shape[0], 2, pages * 16, -1)[:, :, :150])
    a, b = pools
    assert not torch.isnan(a).any() and not torch.isnan(b).any()
    first_layer_differs = float((a[0] != b[0]).float().mean())
    assert first_layer_differs <= 0.01, first_layer_differs       # same inputs: only rounding boundaries
    step = torch.maximum(a[0].abs(), b[0].abs()) * 2.0 ** -7           # one step of bfloat16 at that size
    assert bool(((a[0] - b[0]).abs() <= step + 1e-30).all())
    # later layers read hidden states that already differ by such steps: bounded like the logits
    assert float((a - b).abs().max()) <= TOL_BF16 * max(1.0, float(a.abs().max()))


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


@pytest.mark.parametrize("stored,dtype", [("float32", "float32"), ("bfloat16", "float32"), ("bfloat16", "bfloat16")])
def test_the_references_fixture_through_the_engine(tmp_path, stored, dtype):
    """The reference's golden fixture as a model folder (dequantised; tied with only lm_head stored;
    rope_theta under rope_parameters): the engine's logits at the prompt's last position against the
    reference's reference_logits.bin under the reference's own gate for this fixture
    (crates/ai-engine-runtime/tests/quant_reference_logits.rs:67-82: 3e-2, argmax 150), and at every position
    against the plain implementation, however the four tokens are cut and whatever runs beside them."""
    d = make_fixture_dir(tmp_path, stored)
    ref_last = fixture_reference_logits().astype(np.float64)
    ids = FIXTURE_PROMPT
    oracle = plain_logits(d, ids, oracle_dtype(dtype))
    other = random_ids(70, 512, 3)
    tol = tol_for(dtype)
    rep = replayer(d, dtype, "Q", max_tokens=256)
    runs = {"whole": whole(rep, "w", ids)}
    runs["three_and_one"] = np.concatenate([
        rep.run_step([dict(id="a", tokens=ids[:3], want=[0, 1, 2])]).numpy(),
        rep.run_step([dict(id="a", tokens=ids[3:], want=[0])], end=["a"]).numpy()]).astype(np.float64)
    runs["two_and_two"] = np.concatenate([
        rep.run_step([dict(id="b", tokens=ids[:2], want=[0, 1])]).numpy(),
        rep.run_step([dict(id="b", tokens=ids[2:], want=[0, 1])], end=["b"]).numpy()]).astype(np.float64)
    out = [rep.run_step([dict(id="o", tokens=other[:40], want=[]), dict(id="c", tokens=ids[:2], want=[0, 1])]).numpy()]
    out.append(rep.run_step([dict(id="c", tokens=ids[2:3], want=[0]), dict(id="o", tokens=other[40:69], want=[])]).numpy())
    out.append(rep.run_step([dict(id="o", tokens=other[69:], want=[]), dict(id="c", tokens=ids[3:], want=[0])],
                            end=["o", "c"]).numpy())
    runs["mixed"] = np.concatenate(out).astype(np.float64)
    for how, got in runs.items():
        assert got.shape == oracle.shape
        assert np.abs(got - oracle).max() <= tol, (how, np.abs(got - oracle).max())
        assert int(got[-1].argmax()) == int(ref_last.argmax()) == 150, how
        if stored == "float32":          # the weights as the reference's Q8 path has them: its own gate
            assert np.abs(got[-1] - ref_last).max() < 3e-2, (how, np.abs(got[-1] - ref_last).max())
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


FULL_SIZE_LAYERS = {
    "llama3_8b": dict(hidden_size=4096, intermediate_size=14336, num_attention_heads=32, num_key_value_heads=8,
                      head_dim=128, tie_word_embeddings=False),
    "llama32_3b": dict(hidden_size=3072, intermediate_size=8192, num_attention_heads=24, num_key_value_heads=8,
                       head_dim=128, tie_word_embeddings=True,
                       rope_scaling=dict(rope_type="llama3", factor=32.0, low_freq_factor=1.0, high_freq_factor=4.0,
                                         original_max_position_embeddings=8192)),
    "llama32_1b": dict(hidden_size=2048, intermediate_size=8192, num_attention_heads=32, num_key_value_heads=8,
                       head_dim=64, tie_word_embeddings=True,
                       rope_scaling=dict(rope_type="llama3", factor=32.0, low_freq_factor=1.0, high_freq_factor=4.0,
                                         original_max_position_embeddings=8192)),
}


# float32 at full width against the float64 plain implementation: the engine sums K = 14,336 products in
# one float32 accumulator in a fixed order.  Measured on a B200, the largest difference of a logit is
# 5.9e-5 with logits up to 6.5 (three layers of Llama-3-8B's sizes), 2.2e-5 at 6.2 (3B), 1.5e-5 at 4.5 (1B):
# 0.9e-5 of the largest logit.  The gate leaves a factor of five above that.
F32_FULL_WIDTH_MEASURED = 1e-5
F32_FULL_WIDTH_TOL = 5 * F32_FULL_WIDTH_MEASURED


@pytest.mark.parametrize("name", sorted(FULL_SIZE_LAYERS))
def test_full_size_layers(tmp_path, name):
    """Layers with the sizes of Llama-3-8B (three of them), Llama-3.2-3B and Llama-3.2-1B (one each; a reduced
    vocabulary keeps the folder small): the kernel configurations that full-size models take — products cut along K, tcgen05
    attention, grouped decode — against the plain implementation: a request whole, in portions and token by
    token, with other requests' tokens in the same steps; one step of more than 64 tokens holds two prompt
    portions and a lone decoded token (library products, the tcgen05 prompt kernel and the decode kernel side by side)."""
    import ai_engine_b200 as aie
    from ai_engine_b200.engine.replay import Replayer

    raw = dict(architectures=["LlamaForCausalLM"], num_hidden_layers=3 if name == "llama3_8b" else 1, vocab_size=4096,
               rope_theta=500000.0, rms_norm_eps=1e-5, max_position_embeddings=8192, **FULL_SIZE_LAYERS[name])
    d = os.path.join(str(tmp_path), name)
    aie.write_random_model(aie.LlamaConfig.from_dict(raw), d, seed=5, dtype="bfloat16")
    seqs = {"x": random_ids(200, 4096, 31), "y": random_ids(70, 4096, 32), "z": random_ids(41, 4096, 33)}
    for dtype, odt in (("bfloat16", torch.float32), ("float32", torch.float64)):
        refs = {k: plain_logits(d, v, odt) for k, v in seqs.items()}
        scale = max(1.0, max(float(np.abs(r).max()) for r in refs.values()))
        tol = TOL_BF16 * scale if dtype == "bfloat16" else F32_FULL_WIDTH_TOL * scale
        rep = Replayer(d, dtype, max_tokens=448, block_size=16)
        got = {k: [] for k in seqs}
        fed = {k: 0 for k in seqs}

        def step(*portions):
            entries = [dict(id=k, tokens=seqs[k][fed[k]:fed[k] + n], want=list(range(n))) for k, n in portions]
            out = rep.run_step(entries).numpy()
            row = 0
            for k, n in portions:
                got[k].append(out[row:row + n])
                fed[k] += n
                row += n

        step(("x", 150), ("z", 30))
        step(("x", 40), ("y", 60), ("z", 1))          # 101 tokens: two portions and a lone decoded token
        for _ in range(10):
            step(("y", 1), ("x", 1), ("z", 1))
        worst = 0.0
        for k in seqs:
            err = np.abs(np.concatenate(got[k]) - refs[k]).max(axis=1)
            worst = max(worst, float(err.max()))
            assert err.max() <= tol, (f"{dtype}, request {k}: first wrong token {int(np.argmax(err > tol))}: "
                                      f"{err.max()} (gate {tol}, logits up to {scale})")
        print(f"full-size layers {name} {dtype}: largest difference {worst:.3e} (gate {tol:.3e}, logits up to {scale:.2f})")


def test_the_real_vocabulary_of_llama3_8b(tmp_path):
    """One layer of Llama-3-8B's sizes with its real vocabulary of 128,256 (untied: a 1 GB embedding and a 1 GB
    head of 1,002 weight tiles, the one product of a decode step that is not cut along K): logits rows of a
    prompt portion, of a mixed step and of decoded tokens against the plain implementation, in both dtypes."""
    import ai_engine_b200 as aie
    from ai_engine_b200.engine.replay import Replayer

    raw = dict(architectures=["LlamaForCausalLM"], num_hidden_layers=1, vocab_size=128256, rope_theta=500000.0,
               rms_norm_eps=1e-5, max_position_embeddings=8192, **FULL_SIZE_LAYERS["llama3_8b"])
    d = os.path.join(str(tmp_path), "vocab128256")
    aie.write_random_model(aie.LlamaConfig.from_dict(raw), d, seed=6, dtype="bfloat16")
    rng = np.random.RandomState(3)
    ids = [int(t) for t in rng.randint(0, 128256, size=28)]
    ids[3], ids[20] = 128255, 0                       # the table's last and first rows
    other = [int(t) for t in rng.randint(0, 128256, size=9)]
    ref, ref_other = plain_logits(d, ids, torch.float32), plain_logits(d, other, torch.float32)
    scale = max(1.0, float(np.abs(ref).max()))
    for dtype, tol in (("bfloat16", TOL_BF16 * scale), ("float32", F32_FULL_WIDTH_TOL * scale)):
        rep = Replayer(d, dtype, max_tokens=128, block_size=16)
        got = [rep.run_step([dict(id="x", tokens=ids[:20], want=[0, 3, 19])]).numpy()]
        out = rep.run_step([dict(id="x", tokens=[ids[20]], want=[0]), dict(id="y", tokens=other, want=[8])]).numpy()
        got.append(out[:1])
        for t in ids[21:]:
            got.append(rep.run_step([dict(id="x", tokens=[t], want=[0])]).numpy())
        g = np.concatenate(got)
        assert g.shape == (3 + 1 + 7, 128256)
        err = np.abs(g - ref[[0, 3, 19] + list(range(20, 28))]).max(axis=1)
        assert err.max() <= tol, f"{dtype}: {err} (gate {tol})"
        assert np.abs(out[1] - ref_other[8]).max() <= tol
        del rep
        torch.cuda.empty_cache()


ODD_SIZES = {
    "width_100_head_16": dict(hidden_size=100, intermediate_size=116, num_attention_heads=5, num_key_value_heads=5,
                              head_dim=16, vocab_size=257, tie_word_embeddings=False),
    "head_80_vocab_1001": dict(hidden_size=328, intermediate_size=1000, num_attention_heads=2, num_key_value_heads=1,
                               head_dim=80, vocab_size=1001, tie_word_embeddings=True),
    "head_192": dict(hidden_size=576, intermediate_size=136, num_attention_heads=3, num_key_value_heads=3, head_dim=192,
                     vocab_size=130, tie_word_embeddings=False),
    "head_256_width_520": dict(hidden_size=520, intermediate_size=264, num_attention_heads=2, num_key_value_heads=2,
                               head_dim=256, vocab_size=333, tie_word_embeddings=True),
}


@pytest.mark.parametrize("name", sorted(ODD_SIZES))
def test_sizes_off_the_fast_paths(tmp_path, name):
    """Widths that are no multiple of 8, head sizes that no tensor-core kernel takes, odd vocabularies, plain
    multi-head attention: every size either takes a slower kernel or is refused — never a wrong result."""
    import ai_engine_b200 as aie
    from ai_engine_b200.engine.replay import Replayer

    raw = dict(architectures=["LlamaForCausalLM"], num_hidden_layers=2, rope_theta=10000.0, rms_norm_eps=1e-5,
               max_position_embeddings=512, **ODD_SIZES[name])
    d = os.path.join(str(tmp_path), name)
    aie.write_random_model(aie.LlamaConfig.from_dict(raw), d, seed=9, dtype="bfloat16", std=0.05)
    ids = random_ids(90, raw["vocab_size"], 77)
    ref = plain_logits(d, ids, torch.float32)
    scale = max(1.0, float(np.abs(ref).max()))
    for dtype, tol in (("float32", TOL_F32 * scale), ("bfloat16", TOL_BF16 * scale)):
        rep = Replayer(d, dtype, max_tokens=128, block_size=16)
        got = [rep.run_step([dict(id="x", tokens=ids[:50], want=list(range(50)))]).numpy()]
        got.append(rep.run_step([dict(id="x", tokens=ids[50:83], want=list(range(33)))]).numpy())
        for t in ids[83:]:
            got.append(rep.run_step([dict(id="x", tokens=[t], want=[0])]).numpy())
        err = np.abs(np.concatenate(got) - ref).max(axis=1)
        assert err.max() <= tol, f"{dtype}: first wrong token {int(np.argmax(err > tol))}: {err.max()} (logits up to {scale})"


def test_a_head_size_that_no_kernel_takes_is_refused_by_name(tmp_path):
    import ai_engine_b200 as aie
    from ai_engine_b200.engine.replay import Replayer

    raw = dict(architectures=["LlamaForCausalLM"], num_hidden_layers=1, rope_theta=10000.0, rms_norm_eps=1e-5,
               max_position_embeddings=64, hidden_size=100, intermediate_size=116, num_attention_heads=5,
               num_key_value_heads=5, head_dim=20, vocab_size=257, tie_word_embeddings=False)
    d = os.path.join(str(tmp_path), "head20")
    with pytest.raises(ValueError, match="head_dim 20 must be a multiple of 16"):      # already when the parts are built
        aie.write_random_model(aie.LlamaConfig.from_dict(raw), d, seed=9, dtype="bfloat16")
        Replayer(d, "bfloat16", max_tokens=64, block_size=16)
