"""Typed model configuration: the base class and the config.json reader.

Every architecture has one dataclass whose fields are the keys of its own
``config.json``.  The reference engine never reads config.json and infers the
shape from tensor shapes instead (crates/core/src/weights.rs:62-75, with the
head size fixed at 64 and the norm eps a constant, crates/core/src/config.rs:20);
here every size and constant comes from the file, so no number of the model
stands in code.
"""
from __future__ import annotations

import dataclasses
import json
import os
from typing import Any, ClassVar, Dict, Tuple


class ConfigError(ValueError):
    """config.json is missing, malformed, or describes an impossible model."""


_REQUIRED = object()


def field(key: str | None = None, default: Any = _REQUIRED, doc: str = ""):
    """A dataclass field bound to a config.json key (``key`` defaults to the field name)."""
    meta = {"key": key, "doc": doc}
    if default is _REQUIRED:
        return dataclasses.field(metadata=meta)
    return dataclasses.field(default=default, metadata=meta)


@dataclasses.dataclass
class ModelConfig:
    """Base of all architecture configurations.

    Subclasses declare their fields with :func:`field`; ``from_dict`` fills them
    from a parsed config.json, checks types, and calls ``validate``.
    """

    #: the strings this configuration answers to in config.json's ``architectures``
    architecture_names: ClassVar[Tuple[str, ...]] = ()

    @classmethod
    def from_dict(cls, raw: Dict[str, Any]) -> "ModelConfig":
        if not isinstance(raw, dict):
            raise ConfigError("config.json: top level is not an object")
        kwargs = {}
        problems = []
        for f in dataclasses.fields(cls):
            key = f.metadata.get("key") or f.name
            if key in raw and raw[key] is not None:
                value = raw[key]
                want = _field_type(f)
                try:
                    value = _coerce(value, want)
                except (TypeError, ValueError):
                    problems.append(f"{key}: expected {want.__name__}, got {value!r}")
                    continue
                kwargs[f.name] = value
            elif f.default is dataclasses.MISSING and f.default_factory is dataclasses.MISSING:
                problems.append(f"{key}: required key is missing")
        if problems:
            raise ConfigError("config.json: " + "; ".join(problems))
        cfg = cls(**kwargs)
        cfg.validate()
        return cfg

    def to_dict(self) -> Dict[str, Any]:
        out: Dict[str, Any] = {}
        for f in dataclasses.fields(self):
            out[f.metadata.get("key") or f.name] = getattr(self, f.name)
        return out

    def validate(self) -> None:  # pragma: no cover - overridden
        pass

    @property
    def architecture(self) -> str:
        return self.architecture_names[0]


def _field_type(f: dataclasses.Field) -> type:
    t = f.type
    if isinstance(t, str):
        t = {"int": int, "float": float, "bool": bool, "str": str, "list": list}.get(
            t.replace("Optional[", "").rstrip("]"), object
        )
    return t if isinstance(t, type) else object


def _coerce(value: Any, want: type) -> Any:
    if want is object:
        return value
    if want is bool:
        if isinstance(value, bool):
            return value
        raise TypeError
    if want is int:
        if isinstance(value, bool) or not isinstance(value, int):
            raise TypeError
        return value
    if want is float:
        if isinstance(value, bool) or not isinstance(value, (int, float)):
            raise TypeError
        return float(value)
    if want is str:
        if not isinstance(value, str):
            raise TypeError
        return value
    if want is list:
        if not isinstance(value, list):
            raise TypeError
        return value
    return value


def read_config_json(model_dir: str) -> Dict[str, Any]:
    path = os.path.join(model_dir, "config.json")
    try:
        with open(path, "r", encoding="utf-8") as fh:
            raw = json.load(fh)
    except FileNotFoundError:
        raise ConfigError(f"{path}: no such file") from None
    except json.JSONDecodeError as e:
        raise ConfigError(f"{path}: not valid JSON ({e})") from None
    if not isinstance(raw, dict):
        raise ConfigError(f"{path}: top level is not an object")
    return raw


def architecture_name(raw: Dict[str, Any]) -> str:
    archs = raw.get("architectures")
    if not isinstance(archs, list) or not archs or not isinstance(archs[0], str):
        raise ConfigError("config.json: 'architectures' must be a non-empty list of names")
    return archs[0]
