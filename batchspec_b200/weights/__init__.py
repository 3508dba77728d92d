from .loader import WeightsError, load_weights, random_tensor, random_weights, write_random_model
from .safetensors_io import SafetensorsFile, open_model_files, write_safetensors

__all__ = ["WeightsError", "load_weights", "random_tensor", "random_weights", "write_random_model",
           "SafetensorsFile", "open_model_files", "write_safetensors"]
