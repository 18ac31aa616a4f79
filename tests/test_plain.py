"""The plain implementation itself: the reference's golden fixture, its unit tests
restated (crates/ai-engine-runtime/tests/{rope,norm_and_ffn,sample}.rs), and
properties the formulas imply."""
import math
import os

import numpy as np
import pytest
import torch

import plain_llama as pl
from helpers import (FIXTURE_DIR, FIXTURE_PROMPT, TINY_A, TINY_B, fixture_reference_logits, fixture_tensors,
                     make_model_dir, random_ids)

HERE = os.path.dirname(os.path.abspath(__file__))


def test_golden_fixture_of_the_reference():
    """The reference's reference_logits.bin against the plain implementation, run now, on the reference's
    Q8 fixture (dequantised), under the reference's own Q8 gate
    (crates/ai-engine-runtime/tests/quant_reference_logits.rs:67-82: max |a - b| < 3e-2, equal argmax)."""
    ref = fixture_reference_logits()
    got = pl.forward(fixture_tensors(), pl.read_config(FIXTURE_DIR), FIXTURE_PROMPT)[-1].numpy()
    assert ref.shape == got.shape == (512,)
    assert np.abs(ref - got).max() < 3e-2, np.abs(ref - got).max()
    assert int(ref.argmax()) == int(got.argmax()) == 150
    # float64 changes nothing that the gate could see: the difference is the quantisation's
    w64 = {k: v.double() for k, v in fixture_tensors().items()}
    got64 = pl.forward(w64, pl.read_config(FIXTURE_DIR), FIXTURE_PROMPT)[-1].numpy()
    assert np.abs(got64 - got).max() < 1e-5


def test_llama3_scaling_values():
    """llama3 scaling is not in the reference; the values below were worked out by hand from the rule that
    the config keys name, for head size 8, theta 10000, factor 4, low 1, high 4, original 32: wavelengths
    2*pi / [1, 0.1, 0.01, 0.001] = [6.28, 62.8, 628, 6283]; below 32/4 = 8: kept; above 32/1 = 32: divided
    by 4; (none falls between).  And for original 256: bounds 64 and 256, so 62.8 is kept, 628 and 6283 are
    divided; with original 400 (bounds 100 and 400): 62.8 is kept; with original 100 (bounds 25, 100):
    62.8 lies between: s = (100 / 62.83 - 1) / 3 = 0.19718, value = (1 - s) * 0.1 / 4 + s * 0.1 = 0.039789."""
    sc = lambda orig: dict(rope_type="llama3", factor=4.0, low_freq_factor=1.0, high_freq_factor=4.0,
                           original_max_position_embeddings=orig)
    assert np.allclose(pl.inv_freq_default(8, 10000.0), [1.0, 0.1, 0.01, 0.001], rtol=1e-6)
    assert np.allclose(pl.inv_freq_llama3(8, 10000.0, sc(32)), [1.0, 0.025, 0.0025, 0.00025], rtol=1e-6)
    assert np.allclose(pl.inv_freq_llama3(8, 10000.0, sc(256)), [1.0, 0.1, 0.0025, 0.00025], rtol=1e-6)
    s = (100.0 / (2 * math.pi / 0.1) - 1.0) / 3.0
    assert abs(s - 0.19718) < 1e-5
    assert np.allclose(pl.inv_freq_llama3(8, 10000.0, sc(100)),
                       [1.0, (1 - s) * 0.025 + s * 0.1, 0.0025, 0.00025], rtol=1e-6)
    assert abs(float(pl.inv_freq_llama3(8, 10000.0, sc(100))[1]) - 0.039789) < 1e-6


def test_rope_position_zero_is_identity_and_positions_differ():
    x = torch.randn(2, 3, 16)
    f = pl.inv_freq_default(16, 10000.0)
    assert torch.allclose(pl.rope(x[:, :1], torch.tensor([0]), f), x[:, :1], atol=1e-5)
    a = pl.rope(x[:, :1], torch.tensor([1]), f)
    b = pl.rope(x[:, :1], torch.tensor([5]), f)
    assert not torch.allclose(a, b)
    assert torch.allclose(a.norm(dim=-1), x[:, :1].norm(dim=-1), atol=1e-5)     # a rotation


def test_rope_scores_depend_on_distance_only():
    f = pl.inv_freq_default(32, 500000.0)
    q, k = torch.randn(1, 1, 32, dtype=torch.float64), torch.randn(1, 1, 32, dtype=torch.float64)
    s1 = (pl.rope(q, torch.tensor([7]), f) * pl.rope(k, torch.tensor([3]), f)).sum()
    s2 = (pl.rope(q, torch.tensor([57]), f) * pl.rope(k, torch.tensor([53]), f)).sum()
    assert abs(float(s1 - s2)) < 1e-4


def test_llama3_scaling_by_hand():
    sc = dict(rope_type="llama3", factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0,
              original_max_position_embeddings=64)
    base = pl.inv_freq_default(32, 500000.0).astype(np.float64)
    got = pl.inv_freq_llama3(32, 500000.0, sc).astype(np.float64)
    wl = 2 * math.pi / base
    assert np.allclose(got[wl < 16], base[wl < 16])               # short waves are kept
    assert np.allclose(got[wl > 64], base[wl > 64] / 8.0)         # long waves are stretched
    mid = (wl >= 16) & (wl <= 64)
    assert mid.any() and np.all(got[mid] < base[mid]) and np.all(got[mid] > base[mid] / 8.0)
    assert (wl < 16).any() and (wl > 64).any()


def test_rmsnorm_and_swiglu_by_hand():
    x = torch.tensor([[2.0, 2.0, 2.0, 2.0]])
    assert torch.allclose(pl.rms_norm(x, torch.ones(4), 1e-5), torch.ones(1, 4), atol=1e-5)
    assert torch.allclose(pl.rms_norm(x, torch.tensor([1.0, 2.0, 3.0, 4.0]), 1e-5),
                          torch.tensor([[1.0, 2.0, 3.0, 4.0]]), atol=1e-5)
    h = torch.tensor([[1.0, -2.0]])
    wg, wu, wd = torch.tensor([[1.0, 0.0]]), torch.tensor([[0.0, 1.0]]), torch.tensor([[3.0], [0.5]])
    g, u = 1.0, -2.0
    a = g / (1 + math.exp(-g)) * u
    assert torch.allclose(pl.swiglu(h, wg, wu, wd), torch.tensor([[3.0 * a, 0.5 * a]]), atol=1e-6)


def test_kv_heads_are_repeated_consecutively():
    """4 heads on 2 kv heads: heads 0,1 read kv 0 and heads 2,3 read kv 1
    (crates/ai-engine-runtime/src/arch/attention.rs:177-196)."""
    cfg = dict(heads=4, kv_heads=2, head_dim=4)
    S, D = 3, 8
    torch.manual_seed(0)
    h = torch.randn(S, D)
    wq, wk, wv = torch.randn(16, D), torch.randn(8, D), torch.randn(8, D)
    wo = torch.eye(16)
    f = pl.inv_freq_default(4, 10000.0)
    out = pl.attention(h, wq, wk, wv, wo, torch.arange(S), cfg, f)
    wv2 = wv.clone()
    wv2[4:] = 0                        # silence kv head 1: only heads 2 and 3 may change
    out2 = pl.attention(h, wq, wk, wv2, wo, torch.arange(S), cfg, f)
    assert torch.allclose(out[:, :8], out2[:, :8]) and torch.all(out2[:, 8:] == 0)


def test_logits_at_a_position_do_not_depend_on_later_tokens(tmp_path):
    d = make_model_dir(tmp_path, "B")
    ids = random_ids(30, TINY_B["vocab_size"], 1)
    full = pl.forward_dir(d, ids, torch.float64)
    for n in (1, 2, 9, 17):
        assert torch.allclose(pl.forward_dir(d, ids[:n], torch.float64), full[:n], atol=1e-12)


def test_chosen_rows_are_the_rows_of_the_whole(tmp_path):
    d = make_model_dir(tmp_path, "B")
    ids = random_ids(40, TINY_B["vocab_size"], 2)
    full = pl.forward_dir(d, ids, torch.float64)
    rows = torch.tensor([0, 7, 38, 39])
    assert torch.allclose(pl.forward_dir(d, ids, torch.float64, rows=rows), full[rows], atol=1e-12)


def test_window_masks_old_keys():
    cfg = dict(heads=1, kv_heads=1, head_dim=4)
    torch.manual_seed(1)
    h = torch.randn(6, 4)
    w = [torch.randn(4, 4) for _ in range(3)] + [torch.eye(4)]
    f = pl.inv_freq_default(4, 10000.0)
    full = pl.attention(h, *w, torch.arange(6), cfg, f)
    win = pl.attention(h, *w, torch.arange(6), cfg, f, window=3)
    assert torch.allclose(full[:3], win[:3]) and not torch.allclose(full[5], win[5])
    tail = pl.attention(h[3:], *w, torch.arange(3, 6), cfg, f)       # keys 3..5 only
    assert torch.allclose(win[5], tail[2], atol=1e-6)


def test_sampler_cases():
    """crates/ai-engine-runtime/tests/sample.rs:4-35"""
    logits = [0.1, 2.0, -1.0, 2.0, 0.5]
    assert pl.sample(logits, 0.0) == 1                      # greedy, the first maximum
    assert pl.sample(logits, 1.0, top_k=1, r=0.99) == 1
    assert pl.sample(logits, 1.0, r=0.0) == 1               # the walk starts at the largest
    assert pl.sample(logits, 1.0, r=0.9999999) == 2         # and ends at the smallest
    assert pl.sample([0.0, 10.0, 0.0], 1.0, top_p=0.5, r=0.999) == 1
    counts = np.zeros(5)
    rng = np.random.RandomState(0)
    for _ in range(4000):
        counts[pl.sample(logits, 1.0, r=float(rng.rand()))] += 1
    p = np.exp(logits) / np.exp(logits).sum()
    assert np.abs(counts / 4000 - p).max() < 0.03


def test_read_config_of_both_tiny_models(tmp_path):
    for name, raw in (("A", TINY_A), ("B", TINY_B)):
        cfg = pl.read_config(make_model_dir(tmp_path, name))
        assert cfg["hidden"] == raw["hidden_size"] and cfg["tied"] == raw["tie_word_embeddings"]
        assert (cfg["scaling"] is not None) == ("rope_scaling" in raw)
