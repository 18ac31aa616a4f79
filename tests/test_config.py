"""Configuration and registry (restates crates/ai-engine-runtime/tests/config.rs:17-46)."""
import json
import os

import pytest

import ai_engine_b200 as aie
from ai_engine_b200.config import ConfigError, LlamaConfig, load_config, registered_architectures
from helpers import TINY_A, TINY_B

LLAMA3_8B = dict(architectures=["LlamaForCausalLM"], hidden_size=4096, intermediate_size=14336,
                 num_hidden_layers=32, num_attention_heads=32, num_key_value_heads=8,
                 vocab_size=128256, max_position_embeddings=8192, rope_theta=500000.0,
                 rms_norm_eps=1e-5, tie_word_embeddings=False, eos_token_id=128001)


def test_llama3_8b_parses_and_head_dim_is_derived():
    c = LlamaConfig.from_dict(LLAMA3_8B)
    assert (c.hidden_size, c.num_hidden_layers, c.num_key_value_heads) == (4096, 32, 8)
    assert c.head_dim == 128 and c.eos_token_ids == (128001,)
    assert c.rope_scaling is None and c.tie_word_embeddings is False


def test_defaults_follow_the_reference():
    raw = dict(architectures=["LlamaForCausalLM"], hidden_size=64, intermediate_size=128,
               num_hidden_layers=1, num_attention_heads=4, vocab_size=100)
    c = LlamaConfig.from_dict(raw)
    assert c.num_key_value_heads == 4 and c.head_dim == 16
    assert c.max_position_embeddings == 8192 and c.rope_theta == 10000.0
    assert c.rms_norm_eps == 1e-6 and c.tie_word_embeddings is False


def test_rope_parameters_block_and_llama3_scaling():
    raw = dict(TINY_A)
    del raw["rope_theta"]
    raw["rope_parameters"] = dict(rope_theta=12345.0, rope_type="default")
    assert LlamaConfig.from_dict(raw).rope_theta == 12345.0
    c = LlamaConfig.from_dict(TINY_B)
    assert c.rope_scaling.factor == 8.0 and c.rope_scaling.original_max_position_embeddings == 64
    nested = dict(TINY_B)
    nested["rope_parameters"] = dict(nested.pop("rope_scaling"), rope_theta=nested.pop("rope_theta"))
    assert LlamaConfig.from_dict(nested) == c


def test_round_trip_through_config_json(tmp_path):
    for raw in (TINY_A, TINY_B, LLAMA3_8B):
        c = LlamaConfig.from_dict(raw)
        p = tmp_path / "config.json"
        p.write_text(json.dumps(c.to_dict()))
        arch, c2 = load_config(str(tmp_path))
        assert c2 == c and arch.name == "LlamaForCausalLM"


@pytest.mark.parametrize("change,needle", [
    (dict(architectures=["MixtralForCausalLM"]), "not registered"),
    (dict(architectures=None), "architectures"),
    (dict(hidden_size=None), "hidden_size"),
    (dict(hidden_size="64"), "must be an integer"),
    (dict(intermediate_size=None), "intermediate_size"),
    (dict(num_key_value_heads=3), "multiple"),
    (dict(head_dim=15), "even"),
    (dict(hidden_act="gelu"), "hidden_act"),
    (dict(attention_bias=True), "attention_bias"),
    (dict(rope_scaling=dict(rope_type="yarn", factor=2.0)), "yarn"),
    (dict(rope_scaling=dict(rope_type="llama3", factor=8.0)), "required key"),
    (dict(rms_norm_eps=0.0), "rms_norm_eps"),
    (dict(eos_token_id="x"), "eos_token_id"),
])
def test_bad_configs_are_refused_with_the_key_named(change, needle):
    raw = dict(TINY_A)
    raw.update(change)
    raw = {k: v for k, v in raw.items() if v is not None}
    with pytest.raises(ConfigError) as e:
        load_config(raw)
    assert needle in str(e.value)


def test_registry_lists_what_is_registered():
    assert "LlamaForCausalLM" in registered_architectures()
    with pytest.raises(ConfigError) as e:
        load_config(dict(architectures=["NoSuchModel"]))
    assert "LlamaForCausalLM" in str(e.value)


def test_missing_config_file(tmp_path):
    with pytest.raises(ConfigError):
        load_config(str(tmp_path))


def test_spec_has_no_size_of_its_own():
    """Every size in the built spec comes from the configuration."""
    from ai_engine_b200.models.llama import build_llama_spec

    for raw in (TINY_A, TINY_B):
        c = LlamaConfig.from_dict(raw)
        s = build_llama_spec(c)
        assert len(s.layers) == c.num_hidden_layers and [r.layer for r in s.order] == list(range(len(s.layers)))
        m = s.layers[0].parts["mixer"].params
        assert (m["num_heads"], m["num_kv_heads"], m["head_dim"]) == (
            c.num_attention_heads, c.num_key_value_heads, c.head_dim)
        assert s.layers[0].parts["ffn"].params["intermediate_size"] == c.intermediate_size
        assert s.layers[0].parts["mixer_norm"].params["eps"] == c.rms_norm_eps
        assert s.position_encodings["rope"].params["theta"] == c.rope_theta


def test_rotary_frequencies_by_hand_and_the_fixtures_configuration():
    """The product's frequencies against values worked out by hand (head size 8, theta 10000: 1, 0.1,
    0.01, 0.001; llama3 with factor 4, low 1, high 4: a wavelength below original / 4 is kept, above
    original is divided by 4, between the two blended), and the reference fixture's config.json, whose
    rope_theta is stored under `rope_parameters` only."""
    import math

    import numpy as np

    from ai_engine_b200.parts.rope import rotary_inv_freq
    from helpers import TINY_Q

    sc = lambda orig: dict(rope_type="llama3", factor=4.0, low_freq_factor=1.0, high_freq_factor=4.0,
                           original_max_position_embeddings=orig)
    assert np.allclose(rotary_inv_freq(8, 10000.0), [1.0, 0.1, 0.01, 0.001], rtol=1e-6)
    assert np.allclose(rotary_inv_freq(8, 10000.0, sc(32)), [1.0, 0.025, 0.0025, 0.00025], rtol=1e-6)
    assert np.allclose(rotary_inv_freq(8, 10000.0, sc(256)), [1.0, 0.1, 0.0025, 0.00025], rtol=1e-6)
    s = (100.0 / (2 * math.pi / 0.1) - 1.0) / 3.0
    assert np.allclose(rotary_inv_freq(8, 10000.0, sc(100)), [1.0, (1 - s) * 0.025 + s * 0.1, 0.0025, 0.00025],
                       rtol=1e-6)
    c = LlamaConfig.from_dict(TINY_Q)
    assert (c.rope_theta, c.rope_scaling, c.tie_word_embeddings, c.head_dim, c.eos_token_ids) == (
        10000.0, None, True, 64, (2,))
