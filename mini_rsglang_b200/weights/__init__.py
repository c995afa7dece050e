from .loader import load_weights, open_checkpoint
from .random_init import random_weights, write_random_model
from .safetensors_io import SafetensorsFile, write_safetensors
from .spec import WeightSpec

__all__ = ["load_weights", "open_checkpoint", "random_weights", "write_random_model",
           "SafetensorsFile", "write_safetensors", "WeightSpec"]
