"""Reading and writing model files: safetensors by tensor name, validation against the model's
expected tensors, and the seeded random-weights mode."""
from .safetensors_io import (read_safetensors_header, read_safetensors, write_safetensors,
                             write_sharded_safetensors, TensorFile)
from .loader import ExpectedTensor, LoadedTensors, load_weights, check_tensors, locate_tensors
from .random_init import (normal_values, tensor_key, random_tensors, write_random_model,
                          INIT_MATRIX_STD, INIT_NORM_STD)

__all__ = ["read_safetensors_header", "read_safetensors", "write_safetensors", "write_sharded_safetensors",
           "TensorFile", "ExpectedTensor", "LoadedTensors", "locate_tensors",
           "load_weights", "check_tensors", "normal_values", "tensor_key", "random_tensors",
           "write_random_model", "INIT_MATRIX_STD", "INIT_NORM_STD"]
