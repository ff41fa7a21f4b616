"""What every architecture's typed configuration has in common, and reading a model folder.

The reference keeps its sizes in one pydantic ``ModelParams`` for all of its model families
(torchllms/models/networks.py:110-157) that an offline converter fills from a Hugging Face
``config.json`` (torchllms/models/checkpoint_converter.py:359-397).  Here every architecture has
a configuration class of its own, next to its model description under ``models/``, parsed from
the architecture's own ``config.json`` keys.  This module holds what the framework itself asks
of such a class (:class:`ModelConfig`), the helpers for parsing with errors that name the key,
and the reading of ``config.json`` / ``params.json``.
"""

from __future__ import annotations

import json
from dataclasses import fields, is_dataclass, replace
from pathlib import Path
from typing import Any, Dict, Mapping, Optional, Tuple


class ConfigError(ValueError):
    """A configuration file is missing a key or holds a value that cannot be used."""


def require_key(raw: Mapping[str, Any], key: str, kind, where: str):
    if key not in raw or raw[key] is None:
        raise ConfigError(f"{where}: missing required key '{key}'")
    return typed_value(raw[key], key, kind, where)


def typed_value(value, key: str, kind, where: str):
    if kind is int:
        if isinstance(value, bool) or not isinstance(value, int):
            if isinstance(value, float) and value.is_integer():
                return int(value)
            raise ConfigError(f"{where}: key '{key}' must be an integer, got {value!r}")
        return value
    if kind is float:
        if isinstance(value, bool) or not isinstance(value, (int, float)):
            raise ConfigError(f"{where}: key '{key}' must be a number, got {value!r}")
        return float(value)
    if kind is bool:
        if not isinstance(value, bool):
            raise ConfigError(f"{where}: key '{key}' must be true or false, got {value!r}")
        return value
    if kind is str:
        if not isinstance(value, str):
            raise ConfigError(f"{where}: key '{key}' must be a string, got {value!r}")
        return value
    raise AssertionError(kind)


class ModelConfig:
    """The protocol between an architecture's configuration and the framework.

    A configuration is a frozen dataclass deriving from this class.  The framework reads

    ``architecture``
        the name the architecture is registered under (``config.json``'s ``architectures[0]``);
        random-weight models and written folders are built through it.
    ``max_seq_len``
        the longest sequence the model was made for: the default length of position tables.

    and calls

    ``validate(where)``
        raise :class:`ConfigError` naming the key when a value cannot be used; returns ``self``.
    ``with_overrides(mapping)``
        a copy with fields replaced by name (the reference's ``model_kwargs``,
        torchllms/models/utils.py:53-54).  The default works for any dataclass; a field that
        needs parsing (a nested object given as a dictionary) is handled in ``coerce_override``.
    ``to_hf()``
        the ``config.json`` contents that the architecture's ``parse_config`` reads back to an
        equal object (the random-weights mode writes it).

    Everything else (sizes, constants) is the architecture's own business: only its
    ``build_spec`` reads it.
    """

    architecture: str
    max_seq_len: int

    def validate(self, where: str = "config") -> "ModelConfig":
        return self

    def coerce_override(self, key: str, value: Any) -> Any:
        return value

    def with_overrides(self, overrides: Optional[Mapping[str, Any]]) -> "ModelConfig":
        if not overrides:
            return self
        if not is_dataclass(self):
            raise TypeError(f"{type(self).__name__} must be a dataclass to take overrides")
        known = {f.name for f in fields(self)}
        changed: Dict[str, Any] = {}
        for key, value in overrides.items():
            if key not in known:
                raise ConfigError(f"model_kwargs: unknown configuration field '{key}'")
            changed[key] = self.coerce_override(key, value)
        return replace(self, **changed).validate("model_kwargs")

    def to_hf(self) -> Dict[str, Any]:
        raise NotImplementedError(f"{type(self).__name__} does not say how it is written as config.json")


def read_raw_config(model_dir) -> Tuple[Dict[str, Any], str]:
    """Return the parsed JSON of a model folder and which file it came from."""
    model_dir = Path(model_dir)
    for name in ("config.json", "params.json"):
        path = model_dir / name
        if path.is_file():
            try:
                with open(path) as f:
                    raw = json.load(f)
            except json.JSONDecodeError as e:
                raise ConfigError(f"{path}: not valid JSON ({e})") from None
            if not isinstance(raw, dict):
                raise ConfigError(f"{path}: top level must be an object")
            return raw, name
    raise ConfigError(f"{model_dir}: holds neither config.json nor params.json")
