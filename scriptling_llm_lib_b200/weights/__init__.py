from .loader import WEIGHTS_FILE, WeightError, load_weights
from .random_init import random_tensors, write_random_model
from .safetensors_io import SafetensorsError, SafetensorsFile, write_safetensors
from .spec import TensorSpec

__all__ = ["TensorSpec", "WeightError", "SafetensorsError", "SafetensorsFile", "load_weights", "write_safetensors",
           "random_tensors", "write_random_model", "WEIGHTS_FILE"]
