"""Each part alone against the plain implementation's function of the same name, and
parts that are not Llama's, defined here, registered, built and stepped without a
change to the package: a mixer with state of its own, a layer named twice in the run
order, a layer that reads another's cache, windowed attention in a group of its own."""
import math
from dataclasses import dataclass

import numpy as np
import pytest
import torch

import plain_llama as pl
from helpers import random_ids

pytestmark = pytest.mark.gpu
DEV = "cuda"


def env(dtype, hidden):
    from ai_engine_b200.parts import BuildEnv
    return BuildEnv(hidden, dtype, torch.device(DEV))


def source(tensors, specs, dtype):
    from ai_engine_b200.weights import from_tensors
    return from_tensors(tensors, specs, dtype, DEV)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_rmsnorm_part(dtype):
    from ai_engine_b200.parts import PartSpec, RMSNorm

    D = 200
    p = RMSNorm(PartSpec("rmsnorm", dict(size=D, eps=1e-3), dict(weight="w")), env(dtype, D))
    w = (1 + 0.2 * torch.randn(D)).to(dtype)
    p.load(source({"w": w}, p.tensor_specs(), dtype))
    x = torch.randn(9, D, device=DEV)
    out = p.forward(x.clone())
    want = pl.rms_norm(x.double().cpu(), w.double(), 1e-3)
    assert out.dtype == dtype
    assert (out.double().cpu() - want).abs().max() <= (1e-5 if dtype == torch.float32 else 3e-2)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_swiglu_part(dtype):
    from ai_engine_b200.parts import PartSpec, SwiGLU

    D, F = 72, 200
    p = SwiGLU(PartSpec("swiglu", dict(hidden_size=D, intermediate_size=F), dict(gate="g", up="u", down="d")),
               env(dtype, D))
    ts = {"g": (torch.randn(F, D) * 0.2).to(dtype), "u": (torch.randn(F, D) * 0.2).to(dtype),
          "d": (torch.randn(D, F) * 0.2).to(dtype)}
    p.load(source(ts, p.tensor_specs(), dtype))
    h = torch.randn(11, D).to(dtype)
    out = p.forward(h.to(DEV), None)
    want = pl.swiglu(h.double(), ts["g"].double(), ts["u"].double(), ts["d"].double())
    tol = 1e-5 if dtype == torch.float32 else 5e-2
    assert (out.double().cpu() - want).abs().max() <= tol * max(1.0, float(want.abs().max()))


def test_rotary_part_frequencies():
    from ai_engine_b200.parts import PartSpec, RotaryEncoding

    sc = dict(rope_type="llama3", factor=32.0, low_freq_factor=1.0, high_freq_factor=4.0,
              original_max_position_embeddings=8192)
    for d, theta, scaling in ((16, 10000.0, None), (128, 500000.0, sc), (64, 500000.0, sc)):
        p = RotaryEncoding(PartSpec("rotary", dict(rot_dim=d, theta=theta, scaling=scaling)), env(torch.float32, 8))
        p.load(None)
        want = pl.inv_freq_for(dict(head_dim=d, theta=theta, scaling=scaling))
        assert np.array_equal(p.inv_freq.cpu().numpy(), want)


def tiny_toy_spec(order, layers_kinds, hidden=32, vocab=50, window=0):
    """A model spec from toy and built-in parts (no architecture of anyone's)."""
    from ai_engine_b200.parts import LayerSpec, ModelSpec, PartSpec, RunStep

    layers = []
    for i, kind in enumerate(layers_kinds):
        if kind == "ema":
            mixer = PartSpec("toy_ema", dict(hidden_size=hidden, decay=0.5 + 0.1 * i), dict(w=f"l{i}.mix.w"))
        else:
            mixer = PartSpec("gqa_attention", dict(hidden_size=hidden, num_heads=2, num_kv_heads=1, head_dim=16,
                                                   window=window if kind == "window" else 0, scale=None,
                                                   position_encoding="rope"),
                             dict(q=f"l{i}.q", k=f"l{i}.k", v=f"l{i}.v", o=f"l{i}.o"))
        layers.append(LayerSpec("prenorm", {
            "mixer_norm": PartSpec("rmsnorm", dict(size=hidden, eps=1e-5), dict(weight=f"l{i}.n1")),
            "mixer": mixer,
            "ffn_norm": PartSpec("rmsnorm", dict(size=hidden, eps=1e-5), dict(weight=f"l{i}.n2")),
            "ffn": PartSpec("swiglu", dict(hidden_size=hidden, intermediate_size=48),
                            dict(gate=f"l{i}.g", up=f"l{i}.u", down=f"l{i}.d"))}))
    return ModelSpec(hidden_size=hidden, vocab_size=vocab, max_position=512,
                     embedding=PartSpec("token_embedding", dict(vocab_size=vocab, hidden_size=hidden), dict(weight="emb")),
                     layers=layers, order=[RunStep(*o) if isinstance(o, tuple) else RunStep(o) for o in order],
                     final_norm=PartSpec("rmsnorm", dict(size=hidden, eps=1e-5), dict(weight="fn")),
                     lm_head=PartSpec("lm_head", dict(vocab_size=vocab, hidden_size=hidden), dict(weight="head")),
                     position_encodings={"rope": PartSpec("rotary", dict(rot_dim=16, theta=10000.0, scaling=None))})


def register_toy_mixer():
    """An exponential moving average over a request's tokens: state s <- decay*s + h*w
    per token, output s.  Its state is one [hidden] vector per request, kept in the
    engine's state slots; it has no pages."""
    from ai_engine_b200.parts import Mixer, StateRequest, register_mixer
    from ai_engine_b200.weights import TensorSpec

    class ToyEMA(Mixer):
        host_side = True        # forward walks the requests on the host

        def __init__(self, spec, env):
            super().__init__(spec, env)
            self.hidden, self.decay = int(spec.params["hidden_size"]), float(spec.params["decay"])

        def tensor_specs(self):
            return [TensorSpec(self.spec.tensors["w"], (self.hidden,), init="ones")]

        def load(self, source):
            self.w = source.get(self.spec.tensors["w"]).float()

        def state_request(self):
            return StateRequest((self.hidden,), torch.float32)

        def forward(self, h, ctx, cache):
            out = torch.empty_like(h)
            for r in range(ctx.R):
                slot, a, n = int(ctx.h_slots[r]), int(ctx.h_q_start[r]), int(ctx.h_q_len[r])
                s = cache.state[slot]
                for t in range(a, a + n):
                    s.mul_(self.decay).add_(h[t].float() * self.w)
                    out[t] = s.to(h.dtype)
            return out

    register_mixer("toy_ema", ToyEMA)


def plain_toy_forward(weights, kinds, order, ids, window=0):
    """Whole-sequence float64 restatement of the toy model with the plain functions."""
    w = {k: v.double() for k, v in weights.items()}
    cfg = dict(heads=2, kv_heads=1, head_dim=16)
    f = pl.inv_freq_default(16, 10000.0)
    pos = torch.arange(len(ids))
    x = pl.embed(torch.tensor(ids), w["emb"])
    kv_seen = {}
    for step, o in enumerate(order):
        i, src = (o if isinstance(o, tuple) else (o, None))
        h = pl.rms_norm(x, w[f"l{i}.n1"], 1e-5)
        if kinds[i] == "ema":
            s, outs = torch.zeros(x.shape[1], dtype=torch.float64), []
            for t in range(len(ids)):
                s = (0.5 + 0.1 * i) * s + h[t] * w[f"l{i}.mix.w"]
                outs.append(s)
            a = torch.stack(outs)
        else:
            h_kv = h if src is None else kv_seen[src]
            kv_seen[step] = h_kv
            a = pl_attention_with_kv_from(h, h_kv, w, i, order[src][0] if src is not None and isinstance(order[src], tuple)
                                          else (order[src] if src is not None else i), pos, cfg, f,
                                          window if kinds[i] == "window" else None)
        x = x + a
        h = pl.rms_norm(x, w[f"l{i}.n2"], 1e-5)
        x = x + pl.swiglu(h, w[f"l{i}.g"], w[f"l{i}.u"], w[f"l{i}.d"])
    return pl.rms_norm(x, w["fn"], 1e-5) @ w["head"].T


def pl_attention_with_kv_from(h_q, h_kv, w, i, kv_layer, pos, cfg, f, window):
    """pl.attention, with keys and values projected by layer `kv_layer` from `h_kv`
    (a run that reads another run's cache sees that run's keys and values)."""
    if kv_layer == i and h_q is h_kv:
        return pl.attention(h_q, w[f"l{i}.q"], w[f"l{i}.k"], w[f"l{i}.v"], w[f"l{i}.o"], pos, cfg, f, window)
    S, H, K, d = h_q.shape[0], 2, 1, 16
    q = pl.rope((h_q @ w[f"l{i}.q"].T).view(S, H, d).transpose(0, 1), pos, f)
    k = pl.rope((h_kv @ w[f"l{kv_layer}.k"].T).view(S, K, d).transpose(0, 1), pos, f).expand(H, S, d)
    v = (h_kv @ w[f"l{kv_layer}.v"].T).view(S, K, d).transpose(0, 1).expand(H, S, d)
    sc = (q @ k.transpose(1, 2)) / math.sqrt(d)
    sc = sc.masked_fill(~(pos[None, :] <= pos[:, None])[None], float("-inf"))
    return (torch.softmax(sc, -1) @ v).transpose(0, 1).reshape(S, H * d) @ w[f"l{i}.o"].T


def build_toy(kinds, order, dtype=torch.float32, window=0, seed=0, page=8, pages=24):
    from ai_engine_b200.cache import PagedCache
    from ai_engine_b200.engine.step import StepRunner
    from ai_engine_b200.parts import Model
    from ai_engine_b200.weights import from_tensors, random_tensors

    register_toy_mixer()
    spec = tiny_toy_spec(order, kinds, window=window)
    model = Model(spec, dtype, DEV)
    specs = model.tensor_specs()
    stored = dict(random_tensors(specs, seed, dtype, "cpu", std=0.15, norm_std=0.1))
    model.load(from_tensors(stored, specs, dtype, DEV))
    weights = {k: v.float() for k, v in stored.items()}
    cache = PagedCache(model.cache_requests(), page, pages, 3, 192, dtype, DEV)
    return model, cache, StepRunner(model, cache), weights


def run_in_portions(runner, cache, ids, portions):
    from ai_engine_b200.engine.step import StepEntry

    slot, at, out = cache.admit(), 0, []
    for p in portions:
        assert cache.ensure(slot, at + p)
        out.append(runner.step([StepEntry(slot, at, ids[at:at + p], list(range(p)))]).cpu())
        at += p
        cache.advance(slot, at)
    runner.check_errors()
    cache.finish(slot)
    return torch.cat(out).double()


def test_toy_mixer_with_state_is_registered_built_and_stepped():
    kinds, order = ["ema", "attn", "ema"], [0, 1, 2]
    model, cache, runner, weights = build_toy(kinds, order)
    reqs = model.cache_requests()
    assert [(n.run, n.role, n.kv is not None, n.state is not None) for n in reqs] == [
        (0, "mixer", False, True), (1, "mixer", True, False), (2, "mixer", False, True)]
    assert set(cache.state) == {(0, "mixer"), (2, "mixer")} and len(cache.groups) == 1
    ids = random_ids(40, 50, 3)
    want = plain_toy_forward(weights, kinds, order, ids)
    whole = run_in_portions(runner, cache, ids, [40])
    cut = run_in_portions(runner, cache, ids, [2, 9, 1, 1, 20, 7])
    assert (whole - want).abs().max() <= 1e-4 and (cut - want).abs().max() <= 1e-4
    # two requests side by side keep their own state
    from ai_engine_b200.engine.step import StepEntry
    other = random_ids(12, 50, 4)
    a, b = cache.admit(), cache.admit()
    cache.ensure(a, 40), cache.ensure(b, 12)
    runner.step([StepEntry(a, 0, ids[:30], []), StepEntry(b, 0, other[:5], [])])
    out = runner.step([StepEntry(b, 5, other[5:], [6]), StepEntry(a, 30, ids[30:], [9])]).cpu().double()
    want_b = plain_toy_forward(weights, kinds, order, other)
    assert (out[0] - want_b[11]).abs().max() <= 1e-4 and (out[1] - want[39]).abs().max() <= 1e-4


def test_a_layer_named_twice_and_a_layer_that_reads_anothers_cache():
    kinds = ["attn", "attn"]
    order = [0, 1, 0, (1, 1)]           # layer 0 runs twice (two caches); the last run reads run 1's cache
    model, cache, runner, weights = build_toy(kinds, order, seed=5)
    assert len(cache.groups) == 1 and cache.groups[0].entries == [(0, "mixer"), (1, "mixer"), (2, "mixer")]
    assert cache.where[3, "mixer"] == cache.where[1, "mixer"] and not cache.writes[3, "mixer"]
    ids = random_ids(33, 50, 6)
    want = plain_toy_forward(weights, kinds, order, ids)
    got = run_in_portions(runner, cache, ids, [5, 2, 17, 1, 8])
    assert (got - want).abs().max() <= 1e-4


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_windowed_layers_have_pages_of_their_own_and_give_them_back(dtype):
    kinds, order = ["window", "attn"], [0, 1]
    W = 20
    model, cache, runner, weights = build_toy(kinds, order, dtype=dtype, window=W, seed=7, page=8, pages=20)
    assert len(cache.groups) == 2 and sorted(g.request.window for g in cache.groups) == [0, W]
    ids = random_ids(150, 50, 8)
    want = plain_toy_forward(weights, kinds, order, ids, window=W)
    got = run_in_portions(runner, cache, ids, [33, 2, 40, 1, 1, 1, 30, 42])
    tol = 1e-4 if dtype == torch.float32 else 5e-2
    err = (got - want).abs().max(dim=1).values
    assert err.max() <= tol, f"first wrong token {int((err > tol).nonzero()[0])}"
    wg = [g for g, grp in enumerate(cache.groups) if grp.request.window][0]
    assert cache.book.high_water(wg) <= (42 + W) // 8 + 2       # never the whole sequence
    assert cache.book.high_water(1 - wg) == (150 + 7) // 8


def _step_ctx(cache, slot, start, n, device=DEV):
    """A StepContext for one request bringing tokens [start, start + n) (token ids unused)."""
    from ai_engine_b200.engine.step import StepContext, StepEntry

    err = torch.zeros(1, dtype=torch.int32, device=device)
    return StepContext([StepEntry(slot, start, [0] * n, [])], cache, torch.device(device), err), err


@pytest.mark.parametrize("dtype,H,K,d,window", [(torch.float32, 4, 2, 16, 0), (torch.bfloat16, 6, 2, 64, 0),
                                                (torch.float32, 5, 1, 32, 11), (torch.bfloat16, 8, 8, 128, 0)])
def test_attention_part_alone_over_its_cache(dtype, H, K, d, window):
    """GQAAttention with a rotary encoding, fed in three portions (the last one a single token),
    against plain attention on the whole sequence."""
    from ai_engine_b200.cache import PagedCache
    from ai_engine_b200.parts import BuildEnv, CacheNeed, GQAAttention, PartSpec, RotaryEncoding

    torch.manual_seed(H * d)
    D, S = 96, 45
    e = env(dtype, D)
    rope = RotaryEncoding(PartSpec("rotary", dict(rot_dim=d, theta=500000.0, scaling=None)), e)
    rope.load(None)
    e.position_encodings["rope"] = rope
    part = GQAAttention(PartSpec("gqa_attention", dict(hidden_size=D, num_heads=H, num_kv_heads=K, head_dim=d,
                                                        window=window, scale=None, position_encoding="rope"),
                                 dict(q="q", k="k", v="v", o="o")), e)
    # scores with a standard deviation near 1.5 whatever the head size (as in the tiny configurations),
    # outputs of order 1: bfloat16 rounding then stays inside the bf16 tolerance
    g = (1.5 / D) ** 0.5 / d ** 0.25
    ts = {"q": (torch.randn(H * d, D) * g).to(dtype), "k": (torch.randn(K * d, D) * g).to(dtype),
          "v": (torch.randn(K * d, D) * 0.1).to(dtype), "o": (torch.randn(D, H * d) * 0.06).to(dtype)}
    part.load(source(ts, part.tensor_specs(), dtype))
    cache = PagedCache([CacheNeed(0, "mixer", part.cache_request())], 8, 12, 2, 96, dtype, DEV)
    slot = cache.admit()
    h = torch.randn(S, D).to(dtype)
    outs, at = [], 0
    for n in (30, 14, 1):
        assert cache.ensure(slot, at + n)
        ctx, err = _step_ctx(cache, slot, at, n)
        y = part.forward(h[at:at + n].to(DEV).contiguous(), ctx, cache.part_cache(0, "mixer", ctx)).float()
        outs.append((y.sum(0) if y.dim() == 3 else y).cpu())      # unjoined parts of a split product
        assert int(err.item()) == 0
        at += n
        cache.advance(slot, at)
    got = torch.cat(outs)
    cfg = dict(heads=H, kv_heads=K, head_dim=d)
    want = pl.attention(h.double(), ts["q"].double(), ts["k"].double(), ts["v"].double(), ts["o"].double(),
                        torch.arange(S), cfg, pl.inv_freq_default(d, 500000.0), window or None)
    tol = 1e-4 if dtype == torch.float32 else 3e-2
    err_rows = (got.double() - want).abs().amax(dim=1)
    assert err_rows.max() <= tol, f"first wrong token {int((err_rows > tol).nonzero()[0])}: {float(err_rows.max())}"


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_embedding_and_head_parts(dtype):
    from ai_engine_b200.parts import LMHead, PartSpec, TokenEmbedding

    V, D = 333, 72
    e = env(dtype, D)
    emb = TokenEmbedding(PartSpec("token_embedding", dict(vocab_size=V, hidden_size=D), dict(weight="E")), e)
    head = LMHead(PartSpec("lm_head", dict(vocab_size=V, hidden_size=D), dict(weight="E")), e)     # tied
    table = (torch.randn(V, D) * 0.1).to(dtype)
    src = source({"E": table}, emb.tensor_specs(), dtype)
    emb.load(src)
    head.load(src)
    assert emb.weight.data_ptr() == head.weight.data_ptr()          # one device copy serves both
    ids = torch.tensor([0, 5, 332, 5], dtype=torch.int32, device=DEV)
    err = torch.zeros(1, dtype=torch.int32, device=DEV)
    from types import SimpleNamespace
    x = emb.forward(SimpleNamespace(token_ids=ids, err=err))
    assert x.dtype == torch.float32 and torch.equal(x.cpu(), pl.embed(ids.long().cpu(), table.float()))
    h = torch.randn(3, D).to(dtype)
    logits = head.forward(h.to(DEV), err)
    want = h.double() @ table.double().T
    assert logits.dtype == torch.float32
    assert (logits.double().cpu() - want).abs().max() <= (1e-5 if dtype == torch.float32 else 2e-2)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_prenorm_block_alone(dtype):
    """The block arrangement from its parts against plain decoder_layer: two residuals, the branch
    outputs added inside the following norm."""
    from ai_engine_b200.cache import PagedCache
    from ai_engine_b200.parts import BuildEnv, LayerSpec, PartSpec, RotaryEncoding
    from ai_engine_b200.parts.model import Layer

    torch.manual_seed(4)
    D, H, K, d, F, S = 64, 4, 2, 16, 192, 21
    e = env(dtype, D)
    rope = RotaryEncoding(PartSpec("rotary", dict(rot_dim=d, theta=10000.0, scaling=None)), e)
    rope.load(None)
    e.position_encodings["rope"] = rope
    p = "model.layers.0."
    spec = LayerSpec("prenorm", {
        "mixer_norm": PartSpec("rmsnorm", dict(size=D, eps=1e-5), dict(weight=p + "input_layernorm.weight")),
        "mixer": PartSpec("gqa_attention", dict(hidden_size=D, num_heads=H, num_kv_heads=K, head_dim=d, window=0,
                                                scale=None, position_encoding="rope"),
                          dict(q=p + "self_attn.q_proj.weight", k=p + "self_attn.k_proj.weight",
                               v=p + "self_attn.v_proj.weight", o=p + "self_attn.o_proj.weight")),
        "ffn_norm": PartSpec("rmsnorm", dict(size=D, eps=1e-5), dict(weight=p + "post_attention_layernorm.weight")),
        "ffn": PartSpec("swiglu", dict(hidden_size=D, intermediate_size=F),
                        dict(gate=p + "mlp.gate_proj.weight", up=p + "mlp.up_proj.weight", down=p + "mlp.down_proj.weight"))})
    layer = Layer(spec, e)
    specs = [s for part in layer.parts.values() for s in part.tensor_specs()]
    from ai_engine_b200.weights import random_tensors
    ts = dict(random_tensors(specs, 3, dtype, "cpu", std=0.1, norm_std=0.1))
    src = source(ts, specs, dtype)
    for part in layer.parts.values():
        part.load(src)
    from ai_engine_b200.parts import CacheNeed
    assert [n[0] for n in layer.cache_needs()] == ["mixer"]
    cache = PagedCache([CacheNeed(0, "mixer", layer.parts["mixer"].cache_request())], 8, 8, 1, 64, dtype, DEV)
    slot = cache.admit()
    cache.ensure(slot, S)
    ctx, err = _step_ctx(cache, slot, 0, S)
    x0 = torch.randn(S, D)
    x = x0.clone().to(DEV)
    x, pending = layer.block.forward(x, None, ctx, cache.layer_cache(0, ctx))
    delta = pending.float().sum(0) if pending.dim() == 3 else pending.float()
    got = (x + delta).double().cpu()
    cfg = dict(heads=H, kv_heads=K, head_dim=d, eps=1e-5)
    want = pl.decoder_layer(x0.double(), {k: v.double() for k, v in ts.items()}, 0, torch.arange(S), cfg,
                            pl.inv_freq_default(d, 10000.0))
    assert int(err.item()) == 0
    assert (got - want).abs().max() <= (1e-4 if dtype == torch.float32 else 5e-2)


def test_a_toy_feed_forward_with_routing_is_registered_built_and_stepped():
    """A feed-forward with experts and a router, defined here: router logits and the softmax over the chosen
    experts in float32, the top two of three experts per token, each expert a SwiGLU of the package (the toy
    composes parts; a real one would bring a grouped product).  Registered from outside, chosen for one layer
    of two, fed in portions: the logits are the plain formulas'."""
    from ai_engine_b200.cache import PagedCache
    from ai_engine_b200.engine.step import StepRunner
    from ai_engine_b200.kernels import ops
    from ai_engine_b200.parts import (FeedForward, LayerSpec, Model, ModelSpec, PartSpec, RunStep, SwiGLU,
                                      register_feed_forward)
    from ai_engine_b200.weights import TensorSpec, from_tensors, random_tensors

    E, TOPK, D, F, V = 3, 2, 32, 64, 50

    class ToyRouted(FeedForward):
        def __init__(self, spec, env):
            super().__init__(spec, env)
            self.experts = [SwiGLU(PartSpec("swiglu", dict(hidden_size=D, intermediate_size=F),
                                            {k: f"{spec.tensors['prefix']}.e{e}.{k}" for k in ("gate", "up", "down")}), env)
                            for e in range(E)]

        def tensor_specs(self):
            return [TensorSpec(self.spec.tensors["router"], (E, D))] + [s for x in self.experts for s in x.tensor_specs()]

        def load(self, source):
            self.router = source.get(self.spec.tensors["router"])
            for x in self.experts:
                x.load(source)

        def flops(self, tokens, keys=0.0):
            return 2.0 * tokens * E * D + TOPK * self.experts[0].flops(tokens)

        def forward(self, h, ctx):
            logits = ops.linear(h, self.router, torch.float32, ctx.err)              # [T, E] float32
            top = torch.topk(logits, TOPK, dim=-1)
            gate = torch.softmax(top.values, dim=-1)                                  # float32, over the chosen experts
            out = torch.zeros(h.shape, dtype=torch.float32, device=h.device)
            for e, x in enumerate(self.experts):
                w = (gate * (top.indices == e)).sum(-1)                               # [T]: the token's weight for expert e
                rows = torch.nonzero(w > 0).flatten()
                if rows.numel():
                    y = x.forward(h[rows].contiguous(), ctx)
                    y = y.float().sum(0) if y.dim() == 3 else y.float()
                    out.index_add_(0, rows, y * w[rows, None])
            return out

    register_feed_forward("toy_routed", ToyRouted)
    layers = []
    for i in range(2):
        ffn = (PartSpec("toy_routed", {}, dict(router=f"l{i}.router", prefix=f"l{i}")) if i == 1 else
               PartSpec("swiglu", dict(hidden_size=D, intermediate_size=48), dict(gate=f"l{i}.g", up=f"l{i}.u", down=f"l{i}.d")))
        layers.append(LayerSpec("prenorm", {
            "mixer_norm": PartSpec("rmsnorm", dict(size=D, eps=1e-5), dict(weight=f"l{i}.n1")),
            "mixer": PartSpec("gqa_attention", dict(hidden_size=D, num_heads=2, num_kv_heads=1, head_dim=16, window=0,
                                                    scale=None, position_encoding="rope"),
                              dict(q=f"l{i}.q", k=f"l{i}.k", v=f"l{i}.v", o=f"l{i}.o")),
            "ffn_norm": PartSpec("rmsnorm", dict(size=D, eps=1e-5), dict(weight=f"l{i}.n2")), "ffn": ffn}))
    spec = ModelSpec(hidden_size=D, vocab_size=V, max_position=256,
                     embedding=PartSpec("token_embedding", dict(vocab_size=V, hidden_size=D), dict(weight="emb")),
                     layers=layers, order=[RunStep(0), RunStep(1)],
                     final_norm=PartSpec("rmsnorm", dict(size=D, eps=1e-5), dict(weight="fn")),
                     lm_head=PartSpec("lm_head", dict(vocab_size=V, hidden_size=D), dict(weight="head")),
                     position_encodings={"rope": PartSpec("rotary", dict(rot_dim=16, theta=10000.0, scaling=None))})
    model = Model(spec, torch.float32, DEV)
    specs = model.tensor_specs()
    stored = dict(random_tensors(specs, 4, torch.float32, "cpu", std=0.2, norm_std=0.1))
    model.load(from_tensors(stored, specs, torch.float32, DEV))
    assert model.step_flops(10) > 0 and model.layers[1].parts["ffn"].flops(1) == 2.0 * E * D + TOPK * 2.0 * 3 * F * D
    cache = PagedCache(model.cache_requests(), 8, 16, 2, 128, torch.float32, DEV)
    runner = StepRunner(model, cache)
    ids = random_ids(37, V, 9)
    got = run_in_portions(runner, cache, ids, [5, 2, 17, 1, 12])
    # the plain formulas
    w = {k: v.double() for k, v in stored.items()}
    cfg = dict(heads=2, kv_heads=1, head_dim=16)
    f = pl.inv_freq_default(16, 10000.0)
    pos = torch.arange(len(ids))
    x = pl.embed(torch.tensor(ids), w["emb"])
    for i in range(2):
        h = pl.rms_norm(x, w[f"l{i}.n1"], 1e-5)
        x = x + pl.attention(h, w[f"l{i}.q"], w[f"l{i}.k"], w[f"l{i}.v"], w[f"l{i}.o"], pos, cfg, f)
        h = pl.rms_norm(x, w[f"l{i}.n2"], 1e-5)
        if i == 0:
            x = x + pl.swiglu(h, w["l0.g"], w["l0.u"], w["l0.d"])
        else:
            logits = h @ w["l1.router"].T
            top = torch.topk(logits, TOPK, dim=-1)
            gate = torch.softmax(top.values, dim=-1)
            y = torch.zeros_like(x)
            for t in range(len(ids)):
                for k in range(TOPK):
                    e = int(top.indices[t, k])
                    y[t] += gate[t, k] * pl.swiglu(h[t:t + 1], w[f"l1.e{e}.gate"], w[f"l1.e{e}.up"], w[f"l1.e{e}.down"])[0]
            x = x + y
    want = pl.rms_norm(x, w["fn"], 1e-5) @ w["head"].T
    assert (got - want).abs().max() <= 1e-4, float((got - want).abs().max())
