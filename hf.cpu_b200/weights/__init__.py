from .loader import TensorSpec, WeightError, load_tensors, storage_dtype, weights_path
from .random_init import random_tensors, write_random_model
from .safetensors_io import SafetensorsFile, WeightFormatError, write_safetensors

__all__ = ["TensorSpec", "WeightError", "WeightFormatError", "SafetensorsFile", "load_tensors",
           "storage_dtype", "weights_path", "random_tensors", "write_random_model", "write_safetensors"]
