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

TINY = {"A": (TINY_A, TINY_A_OPTS), "B": (TINY_B, TINY_B_OPTS), "C": (TINY_C, TINY_C_OPTS),
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


def plain_logits(model_dir: str, ids, dtype=torch.float64) -> np.ndarray:
    """[len(ids), vocab] from the plain implementation."""
    return pl.forward_dir(model_dir, ids, dtype).to(torch.float64).numpy()


def random_ids(n: int, vocab: int, seed: int):
    return np.random.RandomState(seed).randint(0, vocab, size=n).tolist()
