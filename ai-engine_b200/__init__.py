"""ai-engine_b200: a single-GPU inference engine for Llama 3 dense models on the
B200 (sm_100a): typed configuration and registry, safetensors weights, layers
from parts, a paged cache, one step function, a scheduler, sampling, and trace
replay, on hand-written CUDA kernels."""
from . import models  # noqa: F401  (registers the architectures)
from .config import ConfigError, LlamaConfig, load_config, register_architecture
from .weights import WeightError, write_random_model

__all__ = ["ConfigError", "LlamaConfig", "load_config", "register_architecture", "WeightError",
           "write_random_model", "Engine", "SamplingParams", "EngineOptions"]


def __getattr__(name):
    if name in ("Engine", "EngineOptions"):
        from .engine import engine as _e
        return getattr(_e, name)
    if name == "SamplingParams":
        from .sampling.params import SamplingParams
        return SamplingParams
    raise AttributeError(name)
