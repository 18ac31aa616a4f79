"""Random weights from a configuration and a seed.

The reference's random mode draws uniform [0,1) matrices and unit norms without
a seed (crates/ai-engine-runtime/src/arch/model.rs:30-34,40-41,79-83), good for
shape tests only.  Here every tensor is drawn from a generator keyed by
(seed, tensor name): matrices N(0, std), norm weights 1 + N(0, norm_std), so a
model folder can be written once and read back by anything that reads
safetensors.
"""
from __future__ import annotations

import hashlib
import json
import os
from typing import Iterator, Sequence, Tuple

import torch

from .loader import TensorSpec
from .safetensors_io import write_safetensors


def _seed_for(seed: int, name: str) -> int:
    h = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    return int.from_bytes(h[:8], "little") & 0x7FFF_FFFF_FFFF_FFFF


def random_tensor(spec: TensorSpec, seed: int, dtype: torch.dtype, device="cpu",
                  std: float = 0.02, norm_std: float = 0.0) -> torch.Tensor:
    g = torch.Generator(device=device)
    g.manual_seed(_seed_for(seed, spec.name))
    if spec.init == "int":
        return torch.randint(0, max(spec.high, 1), spec.shape, generator=g, device=device,
                             dtype=torch.int32)
    if spec.init == "ones":
        t = torch.ones(spec.shape, dtype=torch.float32, device=device)
        if norm_std:
            t += norm_std * torch.randn(spec.shape, generator=g, device=device, dtype=torch.float32)
        return t.to(dtype)
    t = torch.randn(spec.shape, generator=g, device=device, dtype=torch.float32)
    return (t * std).to(dtype)


def random_tensors(specs: Sequence[TensorSpec], seed: int, dtype: torch.dtype, device="cpu",
                   std: float = 0.02, norm_std: float = 0.0) -> Iterator[Tuple[str, torch.Tensor]]:
    for s in specs:
        if s.stored:
            yield s.name, random_tensor(s, seed, dtype, device, std, norm_std)


def write_random_model(config, out_dir: str, seed: int = 0, dtype: str = "bfloat16",
                       std: float = 0.02, norm_std: float = 0.0) -> str:
    """Write `out_dir/config.json` and `out_dir/model.safetensors` for `config`
    (a typed configuration of a registered architecture)."""
    from ..config.registry import resolve_architecture
    from ..parts.model import tensor_specs_of

    raw = config.to_dict()
    arch = resolve_architecture(raw)
    spec = arch.build_spec(config)
    tdt = {"bfloat16": torch.bfloat16, "float32": torch.float32}[dtype]
    os.makedirs(out_dir, exist_ok=True)
    raw["torch_dtype"] = dtype
    with open(os.path.join(out_dir, "config.json"), "w") as f:
        json.dump(raw, f, indent=2)
    write_safetensors(os.path.join(out_dir, "model.safetensors"),
                      random_tensors(tensor_specs_of(spec), seed, tdt, "cpu", std, norm_std),
                      metadata={"format": "pt", "seed": str(seed)})
    return out_dir
