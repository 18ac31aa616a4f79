from .params import SamplingParams
from .rng import philox4x32, uniform

__all__ = ["SamplingParams", "philox4x32", "uniform"]
