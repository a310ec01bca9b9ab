from .qwen3 import Qwen3Config
from .tugelorn import TugelornConfig
from .registry import (Architecture, architecture_of, load_config, read_config_json, register_architecture,
                       registered_architectures)

__all__ = ["Architecture", "Qwen3Config", "TugelornConfig", "architecture_of", "load_config", "read_config_json",
           "register_architecture", "registered_architectures"]
