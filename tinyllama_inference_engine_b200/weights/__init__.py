from .integrity import file_sha256, verify_weights, weights_sha256
from .random_init import random_tensors, write_random_model
from .safetensors_io import SafetensorsFile, write_safetensors
from .store import WeightStore

__all__ = ["SafetensorsFile", "WeightStore", "file_sha256", "random_tensors", "verify_weights", "weights_sha256", "write_random_model", "write_safetensors"]
