from .loader import WeightError, files_have, load_weights
from .random_init import fill_random_, write_random_model
from .safetensors_io import SafetensorsError, SafetensorsFile, open_model_files, save_tensors, write_safetensors

__all__ = [
    "SafetensorsError", "SafetensorsFile", "WeightError", "files_have", "fill_random_", "load_weights",
    "open_model_files", "save_tensors", "write_random_model", "write_safetensors",
]
