from .loader import WeightLoadError, load_weights
from .random_init import fill_random_on_device, random_tensors, write_random_model
from .safetensors_io import SafetensorsFile, write_safetensors

__all__ = [
    "SafetensorsFile", "WeightLoadError", "fill_random_on_device", "load_weights",
    "random_tensors", "write_random_model", "write_safetensors",
]
