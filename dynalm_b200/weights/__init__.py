from .loader import ModelFolder, WeightMismatch, check_tensors, expected_tensors, open_model_folder, place_tensors
from .random_init import random_tensors, write_model_folder
from .safetensors import SafeTensorsFile, write_safetensors

__all__ = ["ModelFolder", "WeightMismatch", "check_tensors", "expected_tensors", "open_model_folder",
           "place_tensors", "random_tensors", "write_model_folder", "SafeTensorsFile", "write_safetensors"]
