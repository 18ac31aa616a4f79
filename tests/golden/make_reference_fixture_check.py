"""Runs the plain implementation (tests/plain_llama.py) on einyx/ai-engine's own
golden fixture and stores both results beside this script.

The fixture is crates/ai-engine-runtime/fixtures/toy-llama-3-q8 in the
reference checkout: int8 Linear weights [out,in] with one f32 `.scale` each,
bf16 norms, no embed_tokens (tied: the embedding is the dequantised lm_head,
crates/ai-engine-runtime/src/loader.rs:129-151), the prompt "The quick brown
fox" -> ids [91, 176, 179, 148] under the fixture's tokenizer.json, and
reference_logits.bin: 512 f32 logits of the last position from the
unquantised bf16 weights run in f32
(crates/ai-engine-runtime/scripts/generate_toy_fixture.py:37-97).  The
reference gates its own Q8 forward on max|a-b| < 3e-2 and an equal argmax
(crates/ai-engine-runtime/tests/quant_reference_logits.rs:67-82).

    python tests/golden/make_reference_fixture_check.py <reference checkout>

writes  toy_q8_reference_logits.f32  (a copy of reference_logits.bin)
        toy_q8_plain_logits.f32      (the plain implementation's logits)
tests/test_plain.py compares the two.
"""
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
import plain_llama as pl  # noqa: E402

PROMPT_IDS = [91, 176, 179, 148]


def main(ref_root: str) -> None:
    fx = os.path.join(ref_root, "crates/ai-engine-runtime/fixtures/toy-llama-3-q8")
    from safetensors import safe_open

    w = {}
    with safe_open(os.path.join(fx, "model.safetensors"), "pt") as f:
        keys = set(f.keys())
        for k in keys:
            if k.endswith(".scale"):
                continue
            t = f.get_tensor(k)
            if t.dtype == torch.int8:
                t = t.to(torch.float32) * f.get_tensor(k + ".scale").to(torch.float32)
            w[k] = t.to(torch.float32)
    cfg = pl.read_config(fx)
    logits = pl.forward(w, cfg, PROMPT_IDS)[-1].numpy().astype("<f4")
    ref = np.fromfile(os.path.join(fx, "reference_logits.bin"), dtype="<f4")
    ref.tofile(os.path.join(HERE, "toy_q8_reference_logits.f32"))
    logits.tofile(os.path.join(HERE, "toy_q8_plain_logits.f32"))
    print("max abs diff", float(np.abs(ref - logits).max()),
          "argmax", int(ref.argmax()), int(logits.argmax()))


if __name__ == "__main__":
    main(sys.argv[1])
