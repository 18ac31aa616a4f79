from .loader import (ModelFolder, TensorSpec, WeightError, WeightSource, check_and_resolve,
                     from_tensors, open_folder)
from .random_init import random_tensor, random_tensors, write_random_model
from .safetensors_io import SafetensorsError, SafetensorsFile, write_safetensors

__all__ = ["ModelFolder", "TensorSpec", "WeightError", "WeightSource", "check_and_resolve",
           "from_tensors", "open_folder", "random_tensor", "random_tensors",
           "write_random_model", "SafetensorsError", "SafetensorsFile", "write_safetensors"]
