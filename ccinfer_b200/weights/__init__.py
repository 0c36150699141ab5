from .loader import (WEIGHTS_FILE, check_tensors, open_weights, random_fetch, random_tensor,
                     write_random_model)
from .safetensors_io import SafetensorsFile, write_safetensors

__all__ = ["SafetensorsFile", "WEIGHTS_FILE", "check_tensors", "open_weights", "random_fetch", "random_tensor",
           "write_random_model", "write_safetensors"]
