from .errors import ConfigError, UnknownArchitectureError
from .reader import KeyReader, read_config_json
from .spec import LayerSpec, ModelSpec, PartSpec
from .mistral import MistralConfig
from .registry import (architecture_names, config_from_dict, load_config,
                       register_architecture)

__all__ = [
    "ConfigError", "UnknownArchitectureError", "KeyReader", "read_config_json",
    "LayerSpec", "ModelSpec", "PartSpec", "MistralConfig", "architecture_names",
    "config_from_dict", "load_config", "register_architecture",
]
