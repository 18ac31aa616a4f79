"""Weights: reading by name, the one error that lists everything wrong, the
random-weights mode (restates crates/ai-engine-runtime/tests/loader.rs:12-48)."""
import json
import os

import numpy as np
import pytest
import torch

import ai_engine_b200 as aie
from ai_engine_b200.config import LlamaConfig
from ai_engine_b200.models.llama import build_llama_spec
from ai_engine_b200.parts import tensor_specs_of
from ai_engine_b200.weights import (ModelFolder, SafetensorsFile, WeightError, check_and_resolve,
                                    from_tensors, write_random_model, write_safetensors)
from helpers import TINY_A, TINY_B


def specs(raw):
    return tensor_specs_of(build_llama_spec(LlamaConfig.from_dict(raw)))


def test_writer_is_read_by_the_safetensors_library_and_back(tmp_path):
    from safetensors import safe_open

    ts = {"a": torch.randn(3, 5), "b": torch.randn(7).bfloat16(), "c": torch.arange(6, dtype=torch.int32).view(2, 3)}
    p = str(tmp_path / "x.safetensors")
    write_safetensors(p, ts.items(), metadata={"k": "v"})
    with safe_open(p, "pt") as f:
        assert set(f.keys()) == set(ts)
        for k in ts:
            assert torch.equal(f.get_tensor(k), ts[k])
    sf = SafetensorsFile(p)
    for k in ts:
        assert torch.equal(sf.tensor(k), ts[k]) and sf.info(k) == (ts[k].dtype, tuple(ts[k].shape))
    assert sf.metadata == {"k": "v"}


def test_random_model_folder_is_seeded_and_complete(tmp_path):
    cfg = LlamaConfig.from_dict(TINY_B)
    d1 = write_random_model(cfg, str(tmp_path / "m1"), seed=1, norm_std=0.1)
    d2 = write_random_model(cfg, str(tmp_path / "m2"), seed=1, norm_std=0.1)
    d3 = write_random_model(cfg, str(tmp_path / "m3"), seed=2, norm_std=0.1)
    f1, f2, f3 = (ModelFolder(d) for d in (d1, d2, d3))
    names = set(f1.names())
    assert "lm_head.weight" not in names and "model.embed_tokens.weight" in names   # tied
    assert len(names) == 2 + 9 * cfg.num_hidden_layers
    for n in names:
        assert torch.equal(f1.tensor(n), f2.tensor(n))
    assert not torch.equal(f1.tensor("model.embed_tokens.weight"), f3.tensor("model.embed_tokens.weight"))
    w = f1.tensor("model.layers.0.mlp.up_proj.weight").float()
    assert abs(float(w.std()) - 0.02) < 2e-3 and w.dtype == torch.float32
    nw = f1.tensor("model.norm.weight").float()
    assert abs(float(nw.mean()) - 1.0) < 0.05 and 0.05 < float(nw.std()) < 0.15
    assert json.load(open(os.path.join(d1, "config.json")))["architectures"] == ["LlamaForCausalLM"]
    check_and_resolve(specs(TINY_B), {n: f1.info(n) for n in names})


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    cfg = LlamaConfig.from_dict(TINY_A)
    d = write_random_model(cfg, str(tmp_path / "m"), seed=0)
    folder = ModelFolder(d)
    avail = {n: folder.info(n) for n in folder.names()}
    del avail["model.layers.1.mlp.down_proj.weight"]
    del avail["lm_head.weight"]
    avail["model.layers.0.self_attn.q_proj.bias"] = (torch.bfloat16, (64,))
    avail["model.layers.7.mlp.up_proj.weight"] = (torch.bfloat16, (192, 64))
    avail["model.layers.0.self_attn.k_proj.weight"] = (torch.bfloat16, (64, 64))
    with pytest.raises(WeightError) as e:
        check_and_resolve(specs(TINY_A), avail, where=d)
    msg = str(e.value)
    assert "missing tensors (2)" in msg and "model.layers.1.mlp.down_proj.weight" in msg and "lm_head.weight" in msg
    assert "unexpected tensors (2)" in msg and "q_proj.bias" in msg and "model.layers.7.mlp.up_proj.weight" in msg
    assert "wrong shapes (1)" in msg and "stored [64, 64], model wants [32, 64]" in msg


def test_tied_embeddings_three_cases():
    """tied head reads the embedding; a tied file with only lm_head serves both;
    untied without lm_head is an error (crates/ai-engine-runtime/src/arch/model.rs:130-134,
    crates/ai-engine-runtime/src/loader.rs:129-151)."""
    sp = specs(TINY_B)
    shapes = {s.name: (torch.bfloat16, s.shape) for s in sp}
    r = check_and_resolve(sp, shapes)
    assert r["model.embed_tokens.weight"] == "model.embed_tokens.weight"
    only_head = dict(shapes)
    only_head["lm_head.weight"] = only_head.pop("model.embed_tokens.weight")
    assert check_and_resolve(sp, only_head)["model.embed_tokens.weight"] == "lm_head.weight"
    spa = specs(TINY_A)
    shapes_a = {s.name: (torch.bfloat16, s.shape) for s in spa}
    del shapes_a["lm_head.weight"]
    with pytest.raises(WeightError) as e:
        check_and_resolve(spa, shapes_a)
    assert "lm_head.weight" in str(e.value)


def test_dtype_policy():
    ts = {"a": torch.randn(4, 4), "b": torch.randn(4, 4).bfloat16(), "c": torch.randn(4, 4).half(),
          "t": torch.arange(4, dtype=torch.int64)}
    from ai_engine_b200.weights import TensorSpec

    sp = [TensorSpec("a", (4, 4)), TensorSpec("b", (4, 4)), TensorSpec("c", (4, 4)), TensorSpec("t", (4,), init="int")]
    src = from_tensors(ts, sp, torch.bfloat16, "cpu")
    assert src.get("a").dtype == torch.float32          # stored in 32-bit stays so
    assert src.get("b").dtype == torch.bfloat16 and src.get("c").dtype == torch.bfloat16
    assert src.get("t").dtype == torch.int32            # integer tables as int32
    src32 = from_tensors(ts, sp, torch.float32, "cpu")
    assert all(src32.get(k).dtype == torch.float32 for k in "abc")


def test_truncated_file_and_missing_folder(tmp_path):
    cfg = LlamaConfig.from_dict(TINY_A)
    d = write_random_model(cfg, str(tmp_path / "m"), seed=0)
    p = os.path.join(d, "model.safetensors")
    data = open(p, "rb").read()
    open(p, "wb").write(data[: len(data) // 2])
    with pytest.raises(WeightError) as e:
        ModelFolder(d)
    assert "truncated" in str(e.value)
    with pytest.raises(WeightError):
        ModelFolder(str(tmp_path / "nothing"))
    os.makedirs(tmp_path / "empty")
    with pytest.raises(WeightError) as e:
        ModelFolder(str(tmp_path / "empty"))
    assert "no *.safetensors" in str(e.value)


def test_integer_stored_weights_are_refused_at_load_by_name(tmp_path):
    """A quantised file (int8 weights with scales beside them, as the reference's Q8 fixture) does not reach
    a kernel: the load fails with the tensors' names (crates/ai-engine-runtime/src/loader.rs:733-750 refuses
    dtypes it does not take at load as well)."""
    import shutil

    from helpers import FIXTURE_DIR
    from ai_engine_b200.config import load_config
    from ai_engine_b200.parts import tensor_specs_of
    from ai_engine_b200.weights import ModelFolder

    d = tmp_path / "q8"
    d.mkdir()
    for f in ("config.json", "model.safetensors"):
        shutil.copy(os.path.join(FIXTURE_DIR, f), d / f)
    arch, cfg = load_config(str(d))
    folder = ModelFolder(str(d))
    available = {n: folder.info(n) for n in folder.names()}
    with pytest.raises(WeightError) as e:
        check_and_resolve(tensor_specs_of(arch.build_spec(cfg)), available)
    msg = str(e.value)
    assert "wrong dtypes (29)" in msg and "lm_head.weight: stored as int8" in msg
    assert "unexpected tensors (29)" in msg and "lm_head.weight.scale" in msg
    folder.close()


def test_buffers_that_are_no_parameters_are_passed_over():
    """An older export stores `rotary_emb.inv_freq` in every layer; the architecture names it as ignorable."""
    from ai_engine_b200.models.llama import build_llama_spec
    from ai_engine_b200.parts import tensor_specs_of

    spec = build_llama_spec(LlamaConfig.from_dict(TINY_A))
    specs = tensor_specs_of(spec)
    available = {s.name: (torch.bfloat16, s.shape) for s in specs}
    available["model.layers.0.self_attn.rotary_emb.inv_freq"] = (torch.float32, (8,))
    check_and_resolve(specs, available, ignored=spec.ignored_tensors)
    with pytest.raises(WeightError, match="unexpected tensors"):
        check_and_resolve(specs, available)
