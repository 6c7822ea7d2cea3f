"""Registries: architecture name -> (config parser, tensor naming); part kind -> class.

The reference picks its model class in C++ in each demo (demo/llama.cpp:119-121) and
has a registry only for kernels (src/op/kernels/kernel_registry.h:29-97).  Here the
model class follows from ``config.json``'s ``architectures[0]`` everywhere: loader,
random-weights writer, engine, trace replay and command line all go through
``architecture()``.

Adding an architecture = one ``register_architecture`` call with
  * ``parse_config(raw: dict) -> ModelConfig``: reads the architecture's own keys;
  * ``tensor_name(scope: tuple, slot: str) -> str``: the safetensors name of a part's
    weight slot.  Scopes are ("embedding",), ("lm_head",), ("final_norm",) and
    ("layer", i, "mixer" | "feed_forward" | "mixer_norm" | "ffn_norm");
  * optionally ``ignored_tensors``: name patterns (fnmatch) of tensors that exporters of this
    architecture store beside the weights and that nothing reads (buffers such as a rotary
    table); the loader passes over them instead of reporting them as unexpected.
Adding a mixer / feed-forward / norm / position encoding / block arrangement = one
``register_part(category, kind, cls)`` call; the class contract is given in
``nanoinfer_b200.parts.base``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Dict, Tuple

from .model_config import ConfigError, ModelConfig, read_config_json

PART_CATEGORIES = ("mixer", "feed_forward", "norm", "position", "arrangement", "embedding", "head")


@dataclass(frozen=True)
class Architecture:
    name: str
    parse_config: Callable[[Dict[str, Any]], ModelConfig]
    tensor_name: Callable[[Tuple, str], str]
    ignored_tensors: Tuple[str, ...] = ()


_ARCHITECTURES: Dict[str, Architecture] = {}
_PARTS: Dict[str, Dict[str, type]] = {c: {} for c in PART_CATEGORIES}


def register_architecture(name: str, parse_config, tensor_name, *, ignored_tensors=(), replace: bool = False) -> None:
    if name in _ARCHITECTURES and not replace:
        raise ConfigError(f"architecture '{name}' is already registered")
    _ARCHITECTURES[name] = Architecture(name, parse_config, tensor_name, tuple(ignored_tensors))


def architecture(name: str) -> Architecture:
    _load_builtin()
    if name not in _ARCHITECTURES:
        known = ", ".join(sorted(_ARCHITECTURES)) or "(none)"
        raise ConfigError(f"unknown architecture '{name}'; registered: {known}")
    return _ARCHITECTURES[name]


def registered_architectures() -> Tuple[str, ...]:
    _load_builtin()
    return tuple(sorted(_ARCHITECTURES))


def register_part(category: str, kind: str, cls: type, *, replace: bool = False) -> None:
    if category not in _PARTS:
        raise ConfigError(f"unknown part category '{category}'; one of {PART_CATEGORIES}")
    if kind in _PARTS[category] and not replace:
        raise ConfigError(f"{category} kind '{kind}' is already registered")
    _PARTS[category][kind] = cls


def part(category: str, kind: str) -> type:
    _load_builtin()
    if category not in _PARTS:
        raise ConfigError(f"unknown part category '{category}'; one of {PART_CATEGORIES}")
    if kind not in _PARTS[category]:
        known = ", ".join(sorted(_PARTS[category])) or "(none)"
        raise ConfigError(f"unknown {category} kind '{kind}'; registered: {known}")
    return _PARTS[category][kind]


def architecture_name_of(raw: Dict[str, Any]) -> str:
    archs = raw.get("architectures")
    if not isinstance(archs, list) or not archs or not isinstance(archs[0], str):
        raise ConfigError("config.json: 'architectures' must be a non-empty list of names")
    return archs[0]


def config_from_dict(raw: Dict[str, Any]) -> ModelConfig:
    """Parse a config.json dictionary with the parser of the architecture it names."""
    arch = architecture(architecture_name_of(raw))
    cfg = arch.parse_config(raw)
    cfg.validate()
    return cfg


def load_config(model_dir: str) -> ModelConfig:
    return config_from_dict(read_config_json(model_dir))


_builtin_loaded = False


def _load_builtin() -> None:
    """Import the modules that register the built-in architecture and parts."""
    global _builtin_loaded
    if _builtin_loaded:
        return
    _builtin_loaded = True
    from .. import parts  # noqa: F401  (registers the part kinds)
    from .. import models  # noqa: F401  (registers architectures)
