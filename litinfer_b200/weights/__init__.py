from .loader import ParamSpec, WeightError, check_against, load_tensors, safetensors_files
from .random_init import random_tensor, random_tensors, write_model_folder
from .safetensors_io import SafetensorsError, iter_tensors, read_header, write_file

__all__ = [
    "ParamSpec",
    "SafetensorsError",
    "WeightError",
    "check_against",
    "iter_tensors",
    "load_tensors",
    "random_tensor",
    "random_tensors",
    "read_header",
    "safetensors_files",
    "write_file",
    "write_model_folder",
]
