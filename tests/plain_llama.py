"""Plain, slow Llama 3 (dense) written from einyx/ai-engine's formulas.

Whole sequences only, no cache, no batching, one function per part, CPU torch.
It shares no code with the product package: it reads model folders with the
`safetensors` library and its own JSON handling, and it is what every engine
test is compared with.

This file rests on the reference's formulas (cited per function by the file's
path within einyx/ai-engine), not on running the reference: the reference is a
Rust workspace and cannot be compiled in the build environment.  Its one
usable anchor is the golden-logits fixture, see tests/golden/.

`dtype` is float32 (what the reference computes in) or float64 (a tighter
truth for the 32-bit engine path).  Rotation angles follow the reference in
both: inv_freq and pos*inv_freq are rounded to float32 first.
"""
from __future__ import annotations

import json
import math
import os

import numpy as np
import torch


# ----------------------------------------------------------------------------
# configuration (its own reading of config.json; keys and defaults as in
# crates/ai-engine-runtime/src/config.rs:22-47,160-184)
# ----------------------------------------------------------------------------
def read_config(model_dir: str) -> dict:
    with open(os.path.join(model_dir, "config.json")) as f:
        raw = json.load(f)
    rp = raw.get("rope_parameters") or {}
    scaling = raw.get("rope_scaling")
    if scaling is None and rp.get("rope_type", "default") not in ("default", None):
        scaling = rp
    cfg = dict(
        hidden=raw["hidden_size"],
        inter=raw["intermediate_size"],
        layers=raw["num_hidden_layers"],
        heads=raw["num_attention_heads"],
        kv_heads=raw.get("num_key_value_heads") or raw["num_attention_heads"],
        head_dim=raw.get("head_dim") or raw["hidden_size"] // raw["num_attention_heads"],
        vocab=raw["vocab_size"],
        theta=float(raw.get("rope_theta", rp.get("rope_theta", 10000.0))),
        eps=float(raw.get("rms_norm_eps", 1e-6)),
        tied=bool(raw.get("tie_word_embeddings", False)),
        scaling=scaling,
    )
    return cfg


def read_weights(model_dir: str, dtype=torch.float32) -> dict:
    from safetensors import safe_open

    out = {}
    for fn in sorted(os.listdir(model_dir)):
        if fn.endswith(".safetensors"):
            with safe_open(os.path.join(model_dir, fn), "pt") as f:
                for k in f.keys():
                    out[k] = f.get_tensor(k).to(dtype)
    return out


# ----------------------------------------------------------------------------
# parts
# ----------------------------------------------------------------------------
def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """crates/ai-engine-runtime/src/arch/rmsnorm.rs:29-42 —
    x * 1/sqrt(mean(x^2) + eps) * w ; eps inside the root, weight last."""
    ms = (x * x).mean(dim=-1, keepdim=True)
    r = 1.0 / torch.sqrt(ms + eps)
    return (x * r) * w


def inv_freq_default(head_dim: int, theta: float) -> np.ndarray:
    """crates/ai-engine-runtime/src/arch/rope.rs:34-36 —
    1 / theta^(2k/d), k in [0, d/2), in f32."""
    k = np.arange(head_dim // 2, dtype=np.float32)
    expo = (np.float32(2.0) * k) / np.float32(head_dim)
    return (np.float32(1.0) / np.power(np.float32(theta), expo)).astype(np.float32)


def inv_freq_llama3(head_dim: int, theta: float, scaling: dict) -> np.ndarray:
    """llama3 rope_scaling.  The reference reads no rope_scaling at all
    (crates/ai-engine-runtime/src/config.rs:22-47 has no such key); this is the
    public rule that the config keys factor / low_freq_factor /
    high_freq_factor / original_max_position_embeddings name: wavelengths
    shorter than original/high stay, longer than original/low are divided by
    factor, and the band between is blended linearly in original/wavelength."""
    base = inv_freq_default(head_dim, theta).astype(np.float64)
    factor = float(scaling["factor"])
    low = float(scaling["low_freq_factor"])
    high = float(scaling["high_freq_factor"])
    orig = float(scaling["original_max_position_embeddings"])
    out = np.empty_like(base)
    for i, f in enumerate(base):
        wavelen = 2.0 * math.pi / f
        if wavelen < orig / high:
            out[i] = f
        elif wavelen > orig / low:
            out[i] = f / factor
        else:
            s = (orig / wavelen - low) / (high - low)
            out[i] = (1.0 - s) * f / factor + s * f
    return out.astype(np.float32)


def inv_freq_for(cfg: dict) -> np.ndarray:
    sc = cfg.get("scaling")
    if sc and (sc.get("rope_type") or sc.get("type")) == "llama3":
        return inv_freq_llama3(cfg["head_dim"], cfg["theta"], sc)
    return inv_freq_default(cfg["head_dim"], cfg["theta"])


def rope(x: torch.Tensor, positions: torch.Tensor, inv_freq: np.ndarray) -> torch.Tensor:
    """crates/ai-engine-runtime/src/arch/rope.rs:38-44,66-106 — split halves:
    out1 = x1*cos - x2*sin ; out2 = x1*sin + x2*cos, angle = f32(pos)*inv_freq
    in f32.  x: [heads, seq, d]."""
    half = x.shape[-1] // 2
    ang32 = positions.to(torch.float32)[:, None] * torch.from_numpy(inv_freq)[None, :]
    ang = ang32.to(x.dtype)
    cos, sin = torch.cos(ang), torch.sin(ang)
    x1, x2 = x[..., :half], x[..., half:]
    return torch.cat([x1 * cos - x2 * sin, x1 * sin + x2 * cos], dim=-1)


def attention(h, wq, wk, wv, wo, positions, cfg, inv_freq, window=None, rows=None) -> torch.Tensor:
    """crates/ai-engine-runtime/src/arch/attention.rs:114-166 (forward),
    :177-196 (consecutive KV-head repeat), :203-224 (mask j <= pos[i]).
    h: [S, D].  `window` (keys j > pos-window only) is not in the reference; it
    serves tests of cache groups with a window.  `rows`: queries are computed for
    these rows of h only (keys and values for all): the same formulas on fewer rows,
    for sequences whose full score matrix would not fit."""
    S = h.shape[0]
    H, K, d = cfg["heads"], cfg["kv_heads"], cfg["head_dim"]
    hq = h if rows is None else h[rows]
    qpos = positions if rows is None else positions[rows]
    Q = hq.shape[0]
    q = (hq @ wq.T).view(Q, H, d).transpose(0, 1)
    k = (h @ wk.T).view(S, K, d).transpose(0, 1)
    v = (h @ wv.T).view(S, K, d).transpose(0, 1)
    q = rope(q, qpos, inv_freq)
    k = rope(k, positions, inv_freq)
    rep = H // K
    k = k[:, None].expand(K, rep, S, d).reshape(H, S, d)
    v = v[:, None].expand(K, rep, S, d).reshape(H, S, d)
    scores = (q @ k.transpose(1, 2)) * (1.0 / math.sqrt(d))
    j = positions[None, :]
    i = qpos[:, None]
    allowed = j <= i
    if window is not None:
        allowed = allowed & (j > i - window)
    scores = scores.masked_fill(~allowed[None], float("-inf"))
    probs = torch.softmax(scores, dim=-1)
    ctx = (probs @ v).transpose(0, 1).reshape(Q, H * d)
    return ctx @ wo.T


def swiglu(h, wg, wu, wd) -> torch.Tensor:
    """crates/ai-engine-runtime/src/arch/ffn.rs:50-54 — down(silu(gate)*up)."""
    g = h @ wg.T
    u = h @ wu.T
    return ((g * torch.sigmoid(g)) * u) @ wd.T


def decoder_layer(x, w: dict, i: int, positions, cfg, inv_freq, rows=None) -> torch.Tensor:
    """crates/ai-engine-runtime/src/arch/block.rs:13-27 — pre-norm, two
    residuals.  `rows`: only these rows of the layer's output are computed and
    returned (their attention still reads every earlier position)."""
    p = f"model.layers.{i}."
    h = rms_norm(x, w[p + "input_layernorm.weight"], cfg["eps"])
    a = attention(h, w[p + "self_attn.q_proj.weight"], w[p + "self_attn.k_proj.weight"],
                  w[p + "self_attn.v_proj.weight"], w[p + "self_attn.o_proj.weight"],
                  positions, cfg, inv_freq, rows=rows)
    x = (x if rows is None else x[rows]) + a
    h = rms_norm(x, w[p + "post_attention_layernorm.weight"], cfg["eps"])
    x = x + swiglu(h, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"],
                   w[p + "mlp.down_proj.weight"])
    return x


def embed(ids: torch.Tensor, table: torch.Tensor) -> torch.Tensor:
    """crates/ai-engine-runtime/src/arch/embedding.rs:14-20 — row gather."""
    return table[ids]


def forward(w: dict, cfg: dict, ids, rows=None) -> torch.Tensor:
    """crates/ai-engine-runtime/src/arch/model.rs:209-224 — embedding, blocks,
    final norm, output projection at every position; tied head uses the
    embedding table (model.rs:130-134), and a file without embed_tokens but
    with lm_head uses that for both (loader.rs:129-151).  Returns [S, V].
    `rows`: logits at these positions only, [len(rows), V]; the last layer, the
    final norm and the head then run on those rows alone (earlier layers need
    every row, since later positions read their keys and values)."""
    ids = torch.as_tensor(ids, dtype=torch.long)
    table = w.get("model.embed_tokens.weight")
    if table is None:
        table = w["lm_head.weight"]
    head = table if cfg["tied"] else w["lm_head.weight"]
    dtype = table.dtype
    positions = torch.arange(ids.shape[0])
    inv_freq = inv_freq_for(cfg)
    x = embed(ids, table)
    for i in range(cfg["layers"]):
        last = i == cfg["layers"] - 1
        x = decoder_layer(x, w, i, positions, cfg, inv_freq, rows=rows if last else None)
    x = rms_norm(x, w["model.norm.weight"], cfg["eps"])
    return (x @ head.T).to(dtype)


def forward_dir(model_dir: str, ids, dtype=torch.float32, rows=None) -> torch.Tensor:
    return forward(read_weights(model_dir, dtype), read_config(model_dir), ids, rows)


# ----------------------------------------------------------------------------
# sampling (crates/ai-engine-runtime/src/sample.rs:12-55)
# ----------------------------------------------------------------------------
def argmax_first(logits) -> int:
    """sample.rs:51-55 — strict '>' so the first maximum wins."""
    best, bv = 0, float("-inf")
    for i, v in enumerate(logits):
        if v > bv:
            best, bv = i, v
    return best


def sample(logits, temperature: float, top_k=None, top_p=None, r: float = 0.0) -> int:
    """sample.rs:12-49 with the uniform draw `r` given from outside: greedy at
    T == 0; else logits/T, sort descending, top-k cut, softmax with the max
    subtracted, top-p cut (shortest prefix with mass >= p, renormalised), walk
    the CDF until r <= acc."""
    logits = [float(x) for x in logits]
    if temperature == 0.0 or len(logits) <= 1:
        return argmax_first(logits)
    scaled = sorted(((np.float32(x) / np.float32(temperature), -i) for i, x in enumerate(logits)),
                    reverse=True)
    probs = [(-negi, x) for x, negi in scaled]
    if top_k is not None:
        probs = probs[:top_k]
    mx = probs[0][1]
    e = [math.exp(float(x - mx)) for _, x in probs]
    s = sum(e)
    p = [v / s for v in e]
    if top_p is not None:
        cum, cut = 0.0, len(p)
        for i, v in enumerate(p):
            cum += v
            if cum >= top_p:
                cut = i + 1
                break
        p = p[:cut]
        probs = probs[:cut]
        s2 = sum(p)
        p = [v / s2 for v in p]
    acc = 0.0
    for (idx, _), v in zip(probs, p):
        acc += v
        if r <= acc:
            return idx
    return probs[-1][0]


def greedy_generate(w: dict, cfg: dict, prompt, n: int) -> list:
    """Whole-sequence recomputation for each new token (no cache)."""
    ids = list(prompt)
    out = []
    for _ in range(n):
        logits = forward(w, cfg, ids)[-1]
        t = int(torch.argmax(logits))
        out.append(t)
        ids.append(t)
    return out
