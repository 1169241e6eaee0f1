from .random_init import random_tensors, write_random_model
from .safetensors_io import SafetensorsFile, write_safetensors
from .store import WeightStore

__all__ = ["SafetensorsFile", "WeightStore", "random_tensors", "write_random_model", "write_safetensors"]
