from .qwen3 import Qwen3Config
from .registry import (Architecture, architecture_of, load_config, read_config_json, register_architecture,
                       registered_architectures)

__all__ = ["Architecture", "Qwen3Config", "architecture_of", "load_config", "read_config_json",
           "register_architecture", "registered_architectures"]
