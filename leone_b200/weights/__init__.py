from .loader import WeightError, check_names_and_shapes, load_checkpoint
from .random_init import random_tensors, write_random_model
from .safetensors import Checkpoint, SafetensorsError, write_safetensors

__all__ = ["WeightError", "check_names_and_shapes", "load_checkpoint", "random_tensors",
           "write_random_model", "Checkpoint", "SafetensorsError", "write_safetensors"]
