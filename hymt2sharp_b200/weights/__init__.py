from .safetensors_io import SafetensorsError, SafetensorsFile, write_safetensors
from .loader import TensorSpec, WeightError, load_checkpoint
from .random_init import write_random_model

__all__ = ["SafetensorsError", "SafetensorsFile", "write_safetensors", "TensorSpec", "WeightError",
           "load_checkpoint", "write_random_model"]
