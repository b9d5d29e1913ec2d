from .loader import WeightsError, check_entries, load_tensors, run_dtype
from .random_init import random_tensors, write_random_model
from .safetensors_io import SafetensorsError, read_header, read_model_headers, read_tensor, write_file

__all__ = ["WeightsError", "check_entries", "load_tensors", "run_dtype", "random_tensors",
           "write_random_model", "SafetensorsError", "read_header", "read_model_headers", "read_tensor",
           "write_file"]
