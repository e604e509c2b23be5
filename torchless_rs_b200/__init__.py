"""torchless_rs_b200: a small model library with generation for one B200, built from
what rglonek/torchless-rs shows for the Mistral dense decoder."""
from .config import (ConfigError, MistralConfig, ModelSpec, LayerSpec, PartSpec,
                     UnknownArchitectureError, config_from_dict, load_config,
                     register_architecture)
from .sampling.params import SamplingParams
from .weights import WeightsMismatchError, write_random_model

__version__ = "0.1.0"

__all__ = ["ConfigError", "MistralConfig", "ModelSpec", "LayerSpec", "PartSpec",
           "UnknownArchitectureError", "config_from_dict", "load_config",
           "register_architecture", "SamplingParams", "WeightsMismatchError",
           "write_random_model", "load", "from_random", "Model"]


def __getattr__(name):
    # the entry points need torch with CUDA and the compiled kernels; import them late so
    # that configuration and weights code can be used without a device
    if name in ("load", "from_random", "Model", "parse_dtype"):
        from . import api
        return getattr(api, name)
    raise AttributeError(name)
