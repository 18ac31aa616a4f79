"""From a model folder (or a configuration and a seed) to a model on the device."""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from ..config.registry import load_config
from ..kernels.loader import require_cuda
from ..parts.model import Model
from ..weights.loader import WeightSource, open_folder
from ..weights.random_init import random_tensor

DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32,
          "fp32": torch.float32, "f32": torch.float32}


def parse_dtype(name) -> torch.dtype:
    if isinstance(name, torch.dtype):
        if name not in (torch.bfloat16, torch.float32):
            raise ValueError(f"compute dtype {name} is not supported (bfloat16, float32)")
        return name
    if name not in DTYPES:
        raise ValueError(f"dtype `{name}` is not supported (bfloat16 | float32)")
    return DTYPES[name]


def load_model(model_dir: str, dtype="bfloat16", device="cuda") -> Tuple[Model, object]:
    """Model class by config.json's architecture, weights by tensor name."""
    require_cuda()
    dt = parse_dtype(dtype)
    arch, cfg = load_config(model_dir)
    model = Model(arch.build_spec(cfg), dt, device)
    source, folder = open_folder(model_dir, model.tensor_specs(), dt, model.device,
                                 ignored=model.spec.ignored_tensors)
    try:
        model.load(source)
    finally:
        source.release()
        folder.close()
    return model, cfg


def random_model(config, seed: int = 0, dtype="bfloat16", device="cuda", std: float = 0.02,
                 norm_std: float = 0.0, num_layers: Optional[int] = None) -> Tuple[Model, object]:
    """A model with random weights drawn on the device, tensor by tensor, without a
    folder (large shapes for measurement).  `config`: a dict in config.json's keys
    or a typed configuration."""
    require_cuda()
    dt = parse_dtype(dtype)
    raw = config if isinstance(config, dict) else config.to_dict()
    arch, cfg = load_config(raw)
    model = Model(arch.build_spec(cfg), dt, device)
    specs = {s.name: s for s in model.tensor_specs()}

    def fetch(name):
        return random_tensor(specs[name], seed, dt, device=model.device, std=std, norm_std=norm_std)

    source = WeightSource(fetch, {n: n for n in specs}, dt, model.device)
    model.load(source)
    source.release()
    return model, cfg
