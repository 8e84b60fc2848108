from .safetensors_io import (SafetensorsError, SafetensorsFile, SafetensorsFolder,
                             save_safetensors)
from .loader import WeightsError, load_weights
from .random_init import random_tensor, random_tensors, write_model_folder

__all__ = ["SafetensorsError", "SafetensorsFile", "SafetensorsFolder", "save_safetensors",
           "WeightsError", "load_weights", "random_tensor", "random_tensors",
           "write_model_folder"]
