from .loader import TensorSpec, WeightError, adopt_tensors, load_weights, storage_dtype
from .random_init import random_tensors, random_weights, write_random_model
from .safetensors_io import Archive, SafetensorsError, Shard, parse_header, write_safetensors

__all__ = ["TensorSpec", "WeightError", "adopt_tensors", "load_weights", "storage_dtype", "random_tensors", "random_weights",
           "write_random_model", "Archive", "SafetensorsError", "Shard", "parse_header",
           "write_safetensors"]
