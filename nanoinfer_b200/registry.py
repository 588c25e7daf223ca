"""The one registry from an architecture's name (config.json's ``architectures[0]``) to its
configuration class and its model builder.

The reference's registry maps names to forward *strategies* (``Stage::spec``,
crates/core/src/stages/mod.rs:157-268, unknown name -> ``Error::UnknownStage``,
crates/core/src/error.rs:17); it knows one architecture only.  Here the registry maps
architectures, so that another one is added by one ``register_architecture`` call.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Dict, Type

from .config.base import ConfigError, ModelConfig, architecture_name, read_config_json
from .models.spec import ModelSpec


@dataclass
class Architecture:
    name: str
    config_cls: Type[ModelConfig]
    build_spec: Callable[[ModelConfig], ModelSpec]


_ARCHITECTURES: Dict[str, Architecture] = {}


class UnknownArchitecture(ConfigError):
    pass


def register_architecture(name: str, config_cls: Type[ModelConfig],
                          build_spec: Callable[[ModelConfig], ModelSpec]) -> None:
    _ARCHITECTURES[name] = Architecture(name, config_cls, build_spec)


def get_architecture(name: str) -> Architecture:
    if name not in _ARCHITECTURES:
        raise UnknownArchitecture(f"unknown architecture {name!r}; registered: {sorted(_ARCHITECTURES)}")
    return _ARCHITECTURES[name]


def architectures():
    return sorted(_ARCHITECTURES)


def load_config(model_dir: str) -> ModelConfig:
    """Read ``model_dir/config.json`` into the typed configuration of its architecture."""
    raw = read_config_json(model_dir)
    arch = get_architecture(architecture_name(raw))
    return arch.config_cls.from_dict(raw)


def _register_builtin() -> None:
    from .config.gpt2 import GPT2Config
    from .models.gpt2 import build_gpt2_spec

    register_architecture("GPT2LMHeadModel", GPT2Config, build_gpt2_spec)


_register_builtin()
