from .loader import (CheckpointSource, TensorSource, TensorSpec, WeightError, find_weight_files, fused_rows,
                     load_tensors, storage_dtype, tensor_meta, weights_path)
from .random_init import RandomSource, random_tensors, write_random_model
from .safetensors_io import SafetensorsFile, WeightFormatError, write_safetensors

__all__ = ["TensorSpec", "TensorSource", "CheckpointSource", "RandomSource", "WeightError", "WeightFormatError",
           "SafetensorsFile", "load_tensors", "find_weight_files", "fused_rows", "tensor_meta", "storage_dtype",
           "weights_path", "random_tensors", "write_random_model", "write_safetensors"]
