"""Shared by the tests: the two tiny Llama configurations (they differ in every
size and option), model folders in a temporary place, and the tolerances."""
from __future__ import annotations

import json
import os

import numpy as np
import torch

import plain_llama as pl

TINY_A = dict(
    architectures=["LlamaForCausalLM"], hidden_size=64, intermediate_size=192,
    num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=16,
    vocab_size=256, rope_theta=10000.0, rms_norm_eps=1e-5, tie_word_embeddings=False,
    max_position_embeddings=128)
# qk_gain scales the q and k projections so that attention scores have a standard
# deviation near 1.6 (0.0256 g^2 for A, 0.064 g^2 for B, 0.038 g^2 for C, 0.077 g^2 for D, 0.102 g^2 for E): single keys
# stand out, and bfloat16 rounding of the scores stays within the bf16 tolerance.
TINY_A_OPTS = dict(seed=0, norm_std=0.0, block_size=16, qk_gain=8.0)

TINY_B = dict(
    architectures=["LlamaForCausalLM"], hidden_size=160, intermediate_size=416,
    num_hidden_layers=3, num_attention_heads=5, num_key_value_heads=1, head_dim=32,
    vocab_size=384, rope_theta=500000.0, rms_norm_eps=1e-6, tie_word_embeddings=True,
    max_position_embeddings=256,
    rope_scaling=dict(rope_type="llama3", factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0,
                      original_max_position_embeddings=64))
TINY_B_OPTS = dict(seed=1, norm_std=0.1, block_size=8, qk_gain=5.0)

# a third shape for long sequences: hundreds of keys, a head size of 48, 6 heads in 3 groups
TINY_C = dict(
    architectures=["LlamaForCausalLM"], hidden_size=96, intermediate_size=160,
    num_hidden_layers=2, num_attention_heads=6, num_key_value_heads=3, head_dim=48,
    vocab_size=200, rope_theta=10000.0, rms_norm_eps=1e-5, tie_word_embeddings=False,
    max_position_embeddings=1024)
TINY_C_OPTS = dict(seed=2, norm_std=0.05, block_size=16, qk_gain=6.0)

# a head size that the fast bfloat16 attention kernels take (64), groups of 3
TINY_D = dict(
    architectures=["LlamaForCausalLM"], hidden_size=192, intermediate_size=272,
    num_hidden_layers=2, num_attention_heads=6, num_key_value_heads=2, head_dim=64,
    vocab_size=300, rope_theta=500000.0, rms_norm_eps=1e-5, tie_word_embeddings=True,
    max_position_embeddings=2048,
    rope_scaling=dict(rope_type="llama3", factor=32.0, low_freq_factor=1.0, high_freq_factor=4.0,
                      original_max_position_embeddings=256))
TINY_D_OPTS = dict(seed=3, norm_std=0.05, block_size=16, qk_gain=4.5)

# head size 128: the tcgen05 attention kernel for prompts and the 128-wide decode kernel
TINY_E = dict(
    architectures=["LlamaForCausalLM"], hidden_size=256, intermediate_size=320,
    num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=128,
    vocab_size=260, rope_theta=500000.0, rms_norm_eps=1e-5, tie_word_embeddings=False,
    max_position_embeddings=2048)
TINY_E_OPTS = dict(seed=4, norm_std=0.05, block_size=16, qk_gain=4.0)

# The reference's own golden fixture (tests/golden/toy-llama-3-q8): 4 layers, 4 heads on 2 kv heads of 64,
# tied with only lm_head stored, rope_theta under rope_parameters; weights dequantised from its int8 file.
FIXTURE_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "toy-llama-3-q8")
FIXTURE_PROMPT = [91, 176, 179, 148]       # "The quick brown fox" under the fixture's tokenizer
with open(os.path.join(FIXTURE_DIR, "config.json")) as _f:
    TINY_Q = json.load(_f)
TINY_Q_OPTS = dict(seed=None, norm_std=None, block_size=16, qk_gain=1.0)

TINY = {"A": (TINY_A, TINY_A_OPTS), "Q": (TINY_Q, TINY_Q_OPTS), "B": (TINY_B, TINY_B_OPTS), "C": (TINY_C, TINY_C_OPTS),
        "D": (TINY_D, TINY_D_OPTS), "E": (TINY_E, TINY_E_OPTS)}

# Tolerances (max abs difference of logits; logits here are O(0.1 .. 1)).
# float32 engine against the float64 plain implementation: the reference's own
# gate for whole prompt against token by token is 1e-4
# (crates/ai-engine-runtime/tests/generation.rs:16-68).
TOL_F32 = 1e-4
# one float32 schedule against another of the same engine
TOL_F32_SCHEDULES = 2e-5
# bfloat16 engine against the float32 plain implementation on the same (bf16)
# weights: the reference's gate for its reduced-precision path is 3e-2
# (crates/ai-engine-runtime/tests/quant_reference_logits.rs:79-82).
TOL_BF16 = 3e-2


def make_model_dir(tmp_path, name: str, dtype: str = "bfloat16", qk_gain=None) -> str:
    """A model folder for tiny configuration `name`, written by the engine's
    random-weights mode.  qk_gain scales the q and k projections so that scores
    spread and single keys stand out (a wrong key or page then changes logits
    far beyond the tolerance)."""
    import ai_engine_b200 as aie

    if name == "Q":
        return make_fixture_dir(tmp_path, dtype)
    raw, opts = TINY[name]
    qk_gain = opts["qk_gain"] if qk_gain is None else qk_gain
    cfg = aie.LlamaConfig.from_dict(raw)
    d = os.path.join(str(tmp_path), f"tiny{name}_{dtype}_{qk_gain}")
    aie.write_random_model(cfg, d, seed=opts["seed"], dtype=dtype, norm_std=opts["norm_std"])
    if qk_gain != 1.0:
        from safetensors import safe_open
        from safetensors.torch import save_file

        path = os.path.join(d, "model.safetensors")
        tensors = {}
        with safe_open(path, "pt") as f:
            for k in f.keys():
                t = f.get_tensor(k)
                if k.endswith("q_proj.weight") or k.endswith("k_proj.weight"):
                    t = (t.float() * qk_gain).to(t.dtype)
                tensors[k] = t.contiguous()
        save_file(tensors, path)
    return d


def fixture_tensors() -> dict:
    """The fixture's tensors in float32: w = int8 * scale for the Linear weights (one float32 scale per
    tensor, stored beside it as `<name>.scale`), the bf16 norms widened
    (crates/ai-engine-runtime/src/loader.rs:733-750 dequantises the same way)."""
    from safetensors import safe_open

    out = {}
    with safe_open(os.path.join(FIXTURE_DIR, "model.safetensors"), "pt") as f:
        for k in f.keys():
            if k.endswith(".scale"):
                continue
            t = f.get_tensor(k)
            if t.dtype == torch.int8:
                t = t.to(torch.float32) * f.get_tensor(k + ".scale").to(torch.float32)
            out[k] = t.to(torch.float32)
    return out


def fixture_reference_logits() -> np.ndarray:
    """The reference's logits at the last position of FIXTURE_PROMPT (512 float32, from the unquantised
    weights: crates/ai-engine-runtime/scripts/generate_toy_fixture.py:37-97)."""
    return np.fromfile(os.path.join(FIXTURE_DIR, "reference_logits.bin"), dtype="<f4")


def make_fixture_dir(tmp_path, dtype: str = "bfloat16") -> str:
    """The fixture as a model folder the engine can load: its config.json as it is, and the
    dequantised tensors stored in `dtype` (no embed_tokens: the tied table is read from lm_head)."""
    from safetensors.torch import save_file

    d = os.path.join(str(tmp_path), f"fixture_{dtype}")
    os.makedirs(d, exist_ok=True)
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(TINY_Q, f)
    dt = dict(bfloat16=torch.bfloat16, float32=torch.float32)[dtype]
    save_file({k: v.to(dt).contiguous() for k, v in fixture_tensors().items()},
              os.path.join(d, "model.safetensors"))
    return d


def plain_logits(model_dir: str, ids, dtype=torch.float64, rows=None) -> np.ndarray:
    """[len(ids), vocab] from the plain implementation ([len(rows), vocab] for chosen rows)."""
    rows = None if rows is None else torch.as_tensor(list(rows), dtype=torch.long)
    return pl.forward_dir(model_dir, ids, dtype, rows).to(torch.float64).numpy()


def random_ids(n: int, vocab: int, seed: int):
    return np.random.RandomState(seed).randint(0, vocab, size=n).tolist()
