"""Configurations drawn at random (from fixed seeds) through the engine against the plain implementation: sizes
that no hand-made tiny configuration has — head sizes in steps of 16 up to 160, groups of 1 to 9 heads, widths and
feed-forward sizes that are multiples of 8 only, odd vocabularies, pages of 8 to 32 keys, llama3 scaling or none,
tied or not — each whole, in portions, and with a second request's tokens in the same steps, in float32 and in
bfloat16.  A size that a kernel does not take must take another kernel or be refused by name, never give other logits.
"""
import numpy as np
import pytest
import torch

from helpers import TOL_BF16, TOL_F32, plain_logits, random_ids

pytestmark = pytest.mark.gpu


def draw(seed):
    r = np.random.RandomState(1000 + seed)
    d = int(r.choice([16, 32, 48, 64, 64, 80, 96, 128, 128, 160]))
    K = int(r.choice([1, 2, 3, 4]))
    G = int(r.choice([1, 2, 3, 4, 5, 8, 9]))
    cfg = dict(architectures=["LlamaForCausalLM"], hidden_size=int(8 * r.randint(6, 40)),
               intermediate_size=int(8 * r.randint(8, 70)), num_hidden_layers=int(r.randint(1, 4)),
               num_attention_heads=K * G, num_key_value_heads=K, head_dim=d,
               vocab_size=int(r.randint(130, 700)), rope_theta=float(r.choice([10000.0, 500000.0])),
               rms_norm_eps=float(r.choice([1e-5, 1e-6])), tie_word_embeddings=bool(r.randint(0, 2)),
               max_position_embeddings=4096)
    if r.randint(0, 2):
        cfg["rope_scaling"] = dict(rope_type="llama3", factor=float(r.choice([8.0, 32.0])), low_freq_factor=1.0,
                                   high_freq_factor=4.0, original_max_position_embeddings=int(r.choice([64, 8192])))
    opts = dict(seed=seed, norm_std=0.05, block_size=int(r.choice([8, 16, 32])), qk_gain=float(r.choice([3.0, 5.0])))
    return cfg, opts


def model_dir(tmp_path, cfg, opts):
    import ai_engine_b200 as aie
    from safetensors import safe_open
    from safetensors.torch import save_file

    d = str(tmp_path / f"random{opts['seed']}")
    aie.write_random_model(aie.LlamaConfig.from_dict(cfg), d, seed=opts["seed"], dtype="bfloat16", norm_std=opts["norm_std"])
    path = d + "/model.safetensors"
    tensors = {}
    with safe_open(path, "pt") as f:
        for k in f.keys():
            t = f.get_tensor(k)
            if k.endswith("q_proj.weight") or k.endswith("k_proj.weight"):
                t = (t.float() * opts["qk_gain"]).to(t.dtype)
            tensors[k] = t.contiguous()
    save_file(tensors, path)
    return d


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("seed", list(range(14)))
def test_a_configuration_drawn_at_random(tmp_path, seed, dtype):
    from ai_engine_b200.engine.replay import Replayer

    cfg, opts = draw(seed)
    d = model_dir(tmp_path, cfg, opts)
    tol = TOL_F32 if dtype == "float32" else TOL_BF16
    odt = torch.float64 if dtype == "float32" else torch.float32
    vocab = cfg["vocab_size"]
    a, b = random_ids(97, vocab, 50 + seed), random_ids(41, vocab, 70 + seed)
    ref_a, ref_b = plain_logits(d, a, odt), plain_logits(d, b, odt)
    what = f"{cfg} pages of {opts['block_size']}"
    rep = Replayer(d, dtype, max_tokens=192, block_size=opts["block_size"], max_num_seqs=4)
    # whole
    got = rep.run_step([dict(id="w", tokens=a, want=list(range(len(a))))], end=["w"]).numpy().astype(np.float64)
    err = np.abs(got - ref_a).max(axis=1)
    assert err.max() <= tol, f"whole: first wrong token {int(np.argmax(err > tol))}: {err.max()} ({what})"
    # request a in portions, request b beside it: first a portion of b, then b token by token
    cuts_a = [3, 17, 2, 30, 1, 1, 9, 34]
    got_a, got_b, at, bt = [], [], 0, 0
    for i, n in enumerate(cuts_a):
        entries = [dict(id="a", tokens=a[at:at + n], want=list(range(n)))]
        m = 20 if i == 0 else (1 if bt < len(b) else 0)
        if i in (3, 7):
            m = min(10, len(b) - bt)
        if m:
            entries.append(dict(id="b", tokens=b[bt:bt + m], want=list(range(m))))
        out = rep.run_step(entries).numpy().astype(np.float64)
        got_a.append(out[:n])
        got_b.append(out[n:])
        at += n
        bt += m
    rep.run_step([], end=["a", "b"])
    got_a, got_b = np.concatenate(got_a), np.concatenate(got_b)
    err = np.abs(got_a - ref_a).max(axis=1)
    assert err.max() <= tol, f"portions: first wrong token {int(np.argmax(err > tol))} of a: {err.max()} ({what})"
    err = np.abs(got_b - ref_b[:bt]).max(axis=1)
    assert err.max() <= tol, f"beside: first wrong token {int(np.argmax(err > tol))} of b: {err.max()} ({what})"
    rep.cache.book.check_invariants()
    assert rep.cache.book.pages_in_use(0) == 0
