from .safetensors_io import SafetensorsError, SafetensorsFile, open_model_files, save_file
from .loader import TensorSpec, WeightsError, canonical_name, load_weights, storage_dtype
from .random_init import random_tensors, write_random_model

__all__ = ["SafetensorsError", "SafetensorsFile", "open_model_files", "save_file", "TensorSpec", "WeightsError",
           "canonical_name", "load_weights", "storage_dtype", "random_tensors", "write_random_model"]
