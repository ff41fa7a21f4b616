"""One registry from an architecture's name to everything that builds its model.

The reference has no such table: it tests substrings of
``config["architectures"][0]`` in its converter
(torchllms/models/checkpoint_converter.py:323-327), checks
``"GptOssForCausalLM" in architectures`` in its driver
(torchllms/inference/llm.py:26-54) and branches on boolean flags in
``Transformer.from_params`` (torchllms/models/networks.py:779-788).  Here the
name that ``config.json`` carries selects an :class:`Architecture`, which
knows how to read the configuration, how to describe the model as data (a
:class:`~torchllms_b200.parts.spec.ModelSpec`), which tensor names a checkpoint
may use, and how to draw random weights.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Dict, Mapping, Optional

from .model_config import ConfigError, read_raw_config


@dataclass(frozen=True)
class Architecture:
    """What the framework needs to know of one model family.

    ``parse_config(raw, source)`` turns the JSON of ``config.json`` (source
    ``"config.json"``) or ``params.json`` into the family's typed configuration.
    ``build_spec(config)`` returns the model as data.  ``adapt_tensors(config,
    tensors)`` maps foreign tensor names (and layouts) to the native ones.
    ``random_tensors(config, seed)`` yields ``(name, tensor)`` in a fixed order.
    ``chat_template`` names the template that conversations are rendered with when the caller
    gives none.  The configuration class derives from
    :class:`~torchllms_b200.config.model_config.ModelConfig`.
    """

    name: str
    parse_config: Callable[[Mapping[str, Any], str], Any]
    build_spec: Callable[[Any], Any]
    adapt_tensors: Callable[[Any, Dict[str, Any]], Dict[str, Any]]
    random_tensors: Callable[..., Any]
    chat_template: Optional[str] = None


ARCHITECTURES: Dict[str, Architecture] = {}


def register_architecture(arch: Architecture) -> Architecture:
    ARCHITECTURES[arch.name] = arch
    return arch


def get_architecture(name: str) -> Architecture:
    _ensure_builtin()
    try:
        return ARCHITECTURES[name]
    except KeyError:
        known = ", ".join(sorted(ARCHITECTURES)) or "(none)"
        raise ConfigError(f"unknown architecture {name!r}; known architectures: {known}") from None


def architecture_of(raw: Mapping[str, Any], source: str) -> Architecture:
    """Pick the architecture that a parsed configuration file names."""
    if source == "params.json":
        # torchllms' own file carries no architecture name; its base
        # Transformer is the Llama decoder unless a flag says otherwise.
        return get_architecture("LlamaForCausalLM")
    archs = raw.get("architectures")
    if not isinstance(archs, (list, tuple)) or not archs or not isinstance(archs[0], str):
        raise ConfigError(f"{source}: missing required key 'architectures' (a list with one name)")
    return get_architecture(archs[0])


def load_config(model_dir, overrides: Optional[Mapping[str, Any]] = None):
    """Read a model folder's configuration; returns ``(architecture, config)``."""
    raw, source = read_raw_config(model_dir)
    arch = architecture_of(raw, source)
    config = arch.parse_config(raw, f"{model_dir}/{source}")
    if overrides:
        config = config.with_overrides(overrides)
    return arch, config


_builtin_loaded = False

PLUGINS_ENV = "TORCHLLMS_B200_PLUGINS"


def _ensure_builtin() -> None:
    """Import every module under ``models/`` (each registers its architecture when imported), then
    the modules that ``TORCHLLMS_B200_PLUGINS`` names (comma separated, importable names): an
    architecture that lives outside the package reaches the command-line programs that way.  A
    program that imports such a module itself needs neither."""
    global _builtin_loaded
    if _builtin_loaded:
        return
    _builtin_loaded = True
    import importlib
    import os
    import pkgutil

    from .. import models
    for info in pkgutil.iter_modules(models.__path__):
        importlib.import_module(f"{models.__name__}.{info.name}")
    for name in filter(None, (n.strip() for n in os.environ.get(PLUGINS_ENV, "").split(","))):
        try:
            importlib.import_module(name)
        except ImportError as e:
            raise ConfigError(f"{PLUGINS_ENV} names module {name!r}, which cannot be imported: {e}") from None
