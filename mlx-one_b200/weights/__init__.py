from .loader import WeightError, check_names, load_weights
from .random_init import random_tensors, write_random_model
from .safetensors_io import SafetensorsError, SafetensorsFile, checkpoint_files, write_safetensors

__all__ = ["WeightError", "check_names", "load_weights", "random_tensors", "write_random_model",
           "SafetensorsError", "SafetensorsFile", "checkpoint_files", "write_safetensors"]
