from .loader import CheckpointFolder, WeightError, bind_weights, check_weights
from .random_init import RandomWeights, random_tensor, write_random_model
from .safetensors_io import SafetensorsError, SafetensorsFile, write_safetensors

__all__ = ["CheckpointFolder", "WeightError", "bind_weights", "check_weights", "RandomWeights", "random_tensor",
           "write_random_model", "SafetensorsError", "SafetensorsFile", "write_safetensors"]
