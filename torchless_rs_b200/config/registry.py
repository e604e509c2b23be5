"""One registry from an architecture's name to its configuration class.

The configuration class turns config.json into a `ModelSpec`; the engine builds
every architecture from its spec with the same code.  The reference maps names
to an enum (src/model/architecture.rs:59-72: "mistral" and "mistralai") and
falls back to Mistral with a warning for unknown names
(src/model/models/mod.rs:93-98); here an unknown name is an error that lists
what is registered.
"""
from __future__ import annotations

from typing import Callable, Dict, List

from .errors import ConfigError, UnknownArchitectureError
from .reader import read_config_json

_ARCHITECTURES: Dict[str, type] = {}


def register_architecture(*names: str) -> Callable[[type], type]:
    """Class decorator: the class must offer `from_dict(dict, where)` and
    `model_spec()`."""
    def deco(cls: type) -> type:
        for n in names:
            _ARCHITECTURES[n.lower()] = cls
        return cls
    return deco


def architecture_names() -> List[str]:
    return sorted(_ARCHITECTURES)


def _name_of(data: dict) -> str:
    archs = data.get("architectures")
    if isinstance(archs, list) and archs and isinstance(archs[0], str):
        return archs[0]
    mt = data.get("model_type")
    if isinstance(mt, str):
        return mt
    raise ConfigError("config.json: neither 'architectures' nor 'model_type' names the architecture")


def config_from_dict(data: dict, where: str = "config.json"):
    name = _name_of(data)
    cls = _ARCHITECTURES.get(name.lower())
    if cls is None:
        raise UnknownArchitectureError(
            f"{where}: architecture '{name}' is not registered; known: {', '.join(architecture_names())}")
    return cls.from_dict(data, where)


def load_config(model_dir: str):
    return config_from_dict(read_config_json(model_dir), where=f"{model_dir}/config.json")


def _register_builtin() -> None:
    from .mistral import MistralConfig
    register_architecture("MistralForCausalLM", "mistral", "mistralai")(MistralConfig)


_register_builtin()
