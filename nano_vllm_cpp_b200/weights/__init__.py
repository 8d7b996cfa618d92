from .safetensors_io import SafetensorsFolder, SafetensorsError, save_safetensors
from .loader import (WeightsError, check_tensors, FolderSource, RandomSource, write_model_folder, load_model)

__all__ = ["SafetensorsFolder", "SafetensorsError", "save_safetensors", "WeightsError", "check_tensors",
           "FolderSource", "RandomSource", "write_model_folder", "load_model"]
