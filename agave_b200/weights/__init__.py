from .safetensors_io import (SafetensorsError, SafetensorsFile, SafetensorsFolder,
                             save_safetensors)
from .loader import LoadedWeights, WeightsError, head_is_stored, load_weights
from .random_init import random_tensor, random_tensors, write_model_folder

__all__ = ["SafetensorsError", "SafetensorsFile", "SafetensorsFolder", "save_safetensors",
           "WeightsError", "LoadedWeights", "head_is_stored", "load_weights", "random_tensor", "random_tensors",
           "write_model_folder"]
