"""A whole toy architecture, defined here and registered from outside the package, run through the
replayer and the engine without a change to the package's files.  It is no model of anyone's; it
exists to use what Llama does not:

* a mixer with state of its own whose update is a CUDA kernel of this folder (tests/toy_parts.cu), under
  captured graphs, with decode batches rounded up by repeated rows (which it must skip), through the engine's
  scheduler with preemption and with the host a step ahead of the device;
* a block with two mixers (attention beside the stateful one), each with a cache of its own;
* an embedding that reads the tokens' positions, and a position encoding that is added to the residual
  stream instead of rotating queries and keys.
"""
import ctypes
import json
import os
from dataclasses import dataclass, field
from typing import List

import numpy as np
import pytest
import torch

import plain_llama as pl
from helpers import TOL_BF16, TOL_F32, random_ids

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))
ARCH = "ToyStatefulForCausalLM"
H, K, HD = 2, 1, 64


@dataclass
class ToyConfig:
    hidden_size: int = 128
    intermediate_size: int = 160
    vocab_size: int = 96
    kinds: List[str] = field(default_factory=lambda: ["ema", "both", "attn"])
    decay: float = 0.6
    max_position_embeddings: int = 512
    eos_token_ids: tuple = ()

    @classmethod
    def from_dict(cls, raw):
        eos = raw.get("eos_token_id") or []
        return cls(raw["hidden_size"], raw["intermediate_size"], raw["vocab_size"], list(raw["kinds"]),
                   float(raw["decay"]), raw["max_position_embeddings"], tuple(eos if isinstance(eos, list) else [eos]))

    def to_dict(self):
        return dict(architectures=[ARCH], hidden_size=self.hidden_size, intermediate_size=self.intermediate_size,
                    vocab_size=self.vocab_size, kinds=self.kinds, decay=self.decay,
                    max_position_embeddings=self.max_position_embeddings, eos_token_id=list(self.eos_token_ids))


def register_toy_architecture():
    import ai_engine_b200 as aie
    from ai_engine_b200.csrc.build import cuda_library
    from ai_engine_b200.kernels import ops
    from ai_engine_b200.kernels.loader import check
    from ai_engine_b200.parts import (Block, LayerSpec, Mixer, ModelSpec, Part, PartSpec, PositionEncoding, RunStep,
                                      StateRequest, register)
    from ai_engine_b200.weights import TensorSpec

    lib = ctypes.CDLL(cuda_library(os.path.join(HERE, "toy_parts.cu")))

    class ToyEMA(Mixer):
        """s <- decay * s + h * w per token, output s; s lives in the request's state slot."""
        skips_padded_rows = True

        def __init__(self, spec, env):
            super().__init__(spec, env)
            self.hidden, self.decay = int(spec.params["hidden_size"]), float(spec.params["decay"])

        def tensor_specs(self):
            return [TensorSpec(self.spec.tensors["w"], (self.hidden,), init="ones")]

        def load(self, source):
            self.w = source.get(self.spec.tensors["w"]).float().contiguous()

        def state_request(self):
            return StateRequest((self.hidden,), torch.float32)

        def forward(self, h, ctx, cache):
            out = torch.empty_like(h)
            p = lambda t: ctypes.c_void_p(t.data_ptr())
            check(lib.toy_ema_scan(p(h), ctypes.c_int(ops.dtype_code(h)), p(self.w), p(cache.state), p(out),
                                   p(ctx.q_start), p(ctx.q_len), p(ctx.slots), p(ctx.live), ctypes.c_int(ctx.R),
                                   ctypes.c_int(self.hidden), ctypes.c_int(cache.state.shape[0]),
                                   ctypes.c_float(self.decay), p(ctx.err), ops._stream()), "toy_ema_scan")
            return out

    class ToyAbsolute(PositionEncoding):
        """A learned table added to the residual stream at each token's position."""

        def tensor_specs(self):
            p = self.spec.params
            return [TensorSpec(self.spec.tensors["table"], (int(p["positions"]), int(p["hidden_size"])))]

        def load(self, source):
            self.table = source.get(self.spec.tensors["table"])

        def add_to(self, x, ctx):
            x.add_(ops.embed_gather(ctx.positions, self.table, ctx.err))

    class ToyPositionEmbedding(Part):
        """E[id] + P[position]: an embedding that reads where the token stands."""

        def tensor_specs(self):
            p = self.spec.params
            return [TensorSpec(self.spec.tensors["weight"], (int(p["vocab_size"]), int(p["hidden_size"]))),
                    TensorSpec(self.spec.tensors["positions"], (int(p["positions"]), int(p["hidden_size"])))]

        def load(self, source):
            self.weight = source.get(self.spec.tensors["weight"])
            self.positions = source.get(self.spec.tensors["positions"])

        def forward(self, ctx):
            x = ops.embed_gather(ctx.token_ids, self.weight, ctx.err)
            return x.add_(ops.embed_gather(ctx.positions, self.positions, ctx.err))

    class TwoMixers(Block):
        """x += attention(norm(x)) + ema(norm(x)); x += ffn(norm(x)): two mixers, a cache each."""
        roles = {"norm": "norm", "attn": "mixer", "ema": "mixer", "ffn_norm": "norm", "ffn": "feed_forward"}

        def __init__(self, spec, env, parts):
            super().__init__(spec, env)
            self.p = parts

        def forward(self, x, pending, ctx, caches):
            h = self.p["norm"].forward(x, pending)
            a = self.p["attn"].forward(h, ctx, caches["attn"])
            b = self.p["ema"].forward(h, ctx, caches["ema"])
            T, D = h.shape
            both = torch.cat([a.float().reshape(-1, T, D), b.float().reshape(1, T, D)])     # the norm adds the parts
            h = self.p["ffn_norm"].forward(x, both)
            return x, self.p["ffn"].forward(h, ctx)

    register("mixer", "toy_ema_cuda", ToyEMA)
    register("position_encoding", "toy_absolute", ToyAbsolute)
    register("embedding", "toy_position_embedding", ToyPositionEmbedding)
    register("block", "toy_two_mixers", TwoMixers)

    def build_spec(cfg: ToyConfig) -> ModelSpec:
        D = cfg.hidden_size
        norm = lambda name: PartSpec("rmsnorm", dict(size=D, eps=1e-5), dict(weight=name))
        layers = []
        for i, kind in enumerate(cfg.kinds):
            attn = PartSpec("gqa_attention", dict(hidden_size=D, num_heads=H, num_kv_heads=K, head_dim=HD, window=0,
                                                  scale=None, position_encoding="rope"),
                            dict(q=f"l{i}.q", k=f"l{i}.k", v=f"l{i}.v", o=f"l{i}.o"))
            ema = PartSpec("toy_ema_cuda", dict(hidden_size=D, decay=cfg.decay), dict(w=f"l{i}.ema.w"))
            ffn = PartSpec("swiglu", dict(hidden_size=D, intermediate_size=cfg.intermediate_size),
                           dict(gate=f"l{i}.g", up=f"l{i}.u", down=f"l{i}.d"))
            if kind == "both":
                layers.append(LayerSpec("toy_two_mixers", {"norm": norm(f"l{i}.n1"), "attn": attn, "ema": ema,
                                                           "ffn_norm": norm(f"l{i}.n2"), "ffn": ffn}))
            else:
                layers.append(LayerSpec("prenorm", {"mixer_norm": norm(f"l{i}.n1"), "mixer": ema if kind == "ema" else attn,
                                                    "ffn_norm": norm(f"l{i}.n2"), "ffn": ffn}))
        return ModelSpec(
            hidden_size=D, vocab_size=cfg.vocab_size, max_position=cfg.max_position_embeddings,
            embedding=PartSpec("toy_position_embedding", dict(vocab_size=cfg.vocab_size, hidden_size=D,
                                                              positions=cfg.max_position_embeddings),
                               dict(weight="emb", positions="emb_pos")),
            layers=layers, order=[RunStep(i) for i in range(len(layers))], final_norm=norm("fn"),
            lm_head=PartSpec("lm_head", dict(vocab_size=cfg.vocab_size, hidden_size=D), dict(weight="head")),
            position_encodings={"rope": PartSpec("rotary", dict(rot_dim=HD, theta=10000.0, scaling=None)),
                                "abs": PartSpec("toy_absolute", dict(positions=cfg.max_position_embeddings, hidden_size=D),
                                                dict(table="abs_pos"))},
            eos_token_ids=cfg.eos_token_ids)

    aie.register_architecture(ARCH, ToyConfig, build_spec)


def toy_dir(tmp_path, eos=()):
    import ai_engine_b200 as aie

    register_toy_architecture()
    d = os.path.join(str(tmp_path), "toy")
    aie.write_random_model(ToyConfig(eos_token_ids=tuple(eos)), d, seed=11, dtype="bfloat16", std=0.08, norm_std=0.1)
    return d


def plain_toy(w, cfg, ids):
    """The toy architecture on a whole sequence with the plain functions (float64)."""
    ids = torch.as_tensor(ids)
    S = ids.shape[0]
    pos = torch.arange(S)
    x = pl.embed(ids, w["emb"]) + w["emb_pos"][pos] + w["abs_pos"][pos]
    acfg = dict(heads=H, kv_heads=K, head_dim=HD)
    f = pl.inv_freq_default(HD, 10000.0)
    for i, kind in enumerate(cfg["kinds"]):
        h = pl.rms_norm(x, w[f"l{i}.n1"], 1e-5)
        a = torch.zeros_like(x)
        if kind in ("attn", "both"):
            a = a + pl.attention(h, w[f"l{i}.q"], w[f"l{i}.k"], w[f"l{i}.v"], w[f"l{i}.o"], pos, acfg, f)
        if kind in ("ema", "both"):
            s, outs = torch.zeros(x.shape[1], dtype=x.dtype), []
            for t in range(S):
                s = cfg["decay"] * s + h[t] * w[f"l{i}.ema.w"]
                outs.append(s)
            a = a + torch.stack(outs)
        x = x + a
        h = pl.rms_norm(x, w[f"l{i}.n2"], 1e-5)
        x = x + pl.swiglu(h, w[f"l{i}.g"], w[f"l{i}.u"], w[f"l{i}.d"])
    return pl.rms_norm(x, w["fn"], 1e-5) @ w["head"].T


def oracle(d, dtype=torch.float64):
    w = pl.read_weights(d, dtype)
    with open(os.path.join(d, "config.json")) as f:
        cfg = json.load(f)
    return w, cfg


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_architecture_replayed_whole_in_portions_and_mixed(tmp_path, dtype):
    from ai_engine_b200.engine.replay import Replayer

    d = toy_dir(tmp_path)
    w, cfg = oracle(d)
    ids, other = random_ids(60, 96, 1), random_ids(45, 96, 2)
    want, want_other = plain_toy(w, cfg, ids).numpy(), plain_toy(w, cfg, other).numpy()
    tol = (TOL_F32 if dtype == "float32" else TOL_BF16) * max(1.0, float(np.abs(want).max()))
    rep = Replayer(d, dtype, max_tokens=256, block_size=16)
    reqs = rep.model.cache_requests()
    assert sorted({n.role for n in reqs}) == ["attn", "ema", "mixer"]
    assert sum(n.state is not None for n in reqs) == 2 and sum(n.kv is not None for n in reqs) == 2
    got = rep.run_step([dict(id="w", tokens=ids, want=list(range(60)))], end=["w"]).numpy()
    assert np.abs(got - want).max() <= tol, np.abs(got - want).max()
    out, at = [], 0
    for n in (2, 9, 1, 1, 20, 7, 1, 19):              # the state after exactly the tokens so far, at every cut
        out.append(rep.run_step([dict(id="p", tokens=ids[at:at + n], want=list(range(n)))]).numpy())
        at += n
    rep.run_step([], end=["p"])
    err = np.abs(np.concatenate(out) - want).max(axis=1)
    assert err.max() <= tol, f"first wrong token {int(np.argmax(err > tol))}: {err.max()}"
    # two requests side by side keep their own state; a slot that is used again starts from zero
    a = rep.run_step([dict(id="x", tokens=ids[:30], want=[29]), dict(id="y", tokens=other[:5], want=[4])]).numpy()
    b = rep.run_step([dict(id="y", tokens=other[5:44], want=[38]), dict(id="x", tokens=[ids[30]], want=[0])]).numpy()
    c = rep.run_step([dict(id="x", tokens=[ids[31]], want=[0]), dict(id="y", tokens=[other[44]], want=[0])],
                     end=["x", "y"]).numpy()
    for g, r in ((a[0], want[29]), (a[1], want_other[4]), (b[0], want_other[43]), (b[1], want[30]), (c[0], want[31]),
                 (c[1], want_other[44])):
        assert np.abs(g - r).max() <= tol


def test_a_captured_step_updates_state_once(tmp_path):
    """Decode steps of one layout: the first runs eagerly, the second runs eagerly and is captured, the
    rest are replayed.  With a mixer that keeps state, every step must update it exactly once: the
    logits are those of the runner that never captures, at every step."""
    from ai_engine_b200.cache import PagedCache
    from ai_engine_b200.engine.loading import load_model
    from ai_engine_b200.engine.step import StepEntry, StepRunner

    d = toy_dir(tmp_path)
    model, _ = load_model(d, "bfloat16")
    assert model.pads_decode_rows() and model.keeps_state() and not model.has_host_parts()
    prompts = [random_ids(20 + 3 * i, 96, 40 + i) for i in range(3)]
    outs = {}
    for graphs in (False, True):
        cache = PagedCache(model.cache_requests(), 16, 32, 4, 512, model.dtype, model.device)
        runner = StepRunner(model, cache, use_graphs=graphs)
        slots = [cache.admit() for _ in prompts]
        for s, p in zip(slots, prompts):
            assert cache.ensure(s, len(p))
            runner.step([StepEntry(s, 0, p[:10], [])])
        got = []
        for k in range(10, 20):
            got.append(runner.step([StepEntry(s, k, [p[k]], [0]) for s, p in zip(slots, prompts)]).float().cpu())
        runner.check_errors()
        outs[graphs] = torch.stack(got)
        if graphs:
            assert runner.graphs_captured == 1 and runner.graph_launches > 0
    assert (outs[True] - outs[False]).abs().max() <= 1e-2
    w, cfg = oracle(d, torch.float32)
    want = plain_toy(w, cfg, prompts[1][:20])[10:20]
    assert (outs[True][:, 1] - want).abs().max() <= TOL_BF16 * max(1.0, float(want.abs().max()))


def greedy_toy(w, cfg, prompt, n):
    ids, out, margins = list(prompt), [], []
    for _ in range(n):
        logits = plain_toy(w, cfg, ids)[-1]
        top = torch.topk(logits, 2).values
        out.append(int(torch.argmax(logits)))
        margins.append(float(top[0] - top[1]))
        ids.append(out[-1])
    return out, margins


def test_engine_serves_the_stateful_toy_model_with_graphs_padded_rows_and_preemption(tmp_path):
    """Twelve requests of mixed lengths on sixteen seats, bfloat16: decode batches wander through 9 .. 12 rows
    (rounded up to 16 by repeated rows, which the stateful mixer must skip) and below 8, from captured
    graphs; with a roomy pool and one so tight that requests are preempted and recomputed (their state
    starts again from zero); with the host a step ahead of the device and not.  Every sequence is the plain
    implementation's greedy continuation until a near-tie."""
    import ai_engine_b200 as aie

    d = toy_dir(tmp_path)
    w, cfg = oracle(d, torch.float32)
    rng = np.random.RandomState(5)
    prompts = [random_ids(int(n), 96, 100 + i) for i, n in enumerate(rng.randint(3, 60, size=12))]
    news = [int(n) for n in rng.randint(6, 30, size=12)]
    params = [aie.SamplingParams(max_tokens=n, ignore_eos=True) for n in news]
    need = sum((len(p) + n + 15) // 16 for p, n in zip(prompts, news))
    outs = {}
    for blocks in (need + 4, need // 2):
        for ahead in (False, True):
            eng = aie.Engine(d, dtype="bf16", block_size=16, kv_cache_blocks=blocks, max_num_seqs=16,
                             max_num_batched_tokens=64, async_scheduling=ahead)
            assert eng.runner.use_graphs and eng.runner.pad_decode
            outs[blocks, ahead] = eng.generate(prompts, params)
            st = eng.stats()
            assert eng.runner.graphs_captured >= 1
            assert all(g["in_use"] == 0 for g in st["cache"].values()) and st["running"] == 0
            assert (st["preemptions"] >= 1) == (blocks < need), (blocks, need, st["preemptions"])
        assert outs[blocks, True] == outs[blocks, False]
    tol = TOL_BF16 * 2
    for key, got in outs.items():
        for p, n, o in zip(prompts, news, got):
            want, margins = greedy_toy(w, cfg, p, n)
            for i, (g, x) in enumerate(zip(o, want)):
                if g != x:
                    assert margins[i] <= tol, f"{key}: token {i}: got {g}, plain {x}, margin {margins[i]}"
                    break
            assert len(o) == n
