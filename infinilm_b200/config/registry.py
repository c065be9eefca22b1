"""One registry from an architecture's name to its configuration class and model description.

Parity with InfiniLM: `csrc/models/models_registry.hpp:22-79` (static map from model_type to
a model creator and a config creator), `csrc/models/model_factory.cpp:6-26` (unknown name is
an `invalid_argument`). Lookup tries `architectures[0]`, then `model_type`.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Dict, Iterable, List

from .model_config import ConfigError, ModelConfig, read_config_json


@dataclass
class Architecture:
    names: List[str]
    config_cls: type
    describe: Callable[[ModelConfig], Any]      # ModelConfig -> parts.spec.ModelSpec


_ARCHITECTURES: Dict[str, Architecture] = {}


def register_architecture(names: Iterable[str], config_cls: type,
                          describe: Callable[[ModelConfig], Any]) -> Architecture:
    """Make an architecture known under each of `names` (HF class name, model_type...).

    `config_cls.from_json(dict)` must return a `ModelConfig`; `describe(config)` must return the
    model's description (`ModelSpec`): its parts layer by layer and the order they run in."""
    arch = Architecture(list(names), config_cls, describe)
    for n in arch.names:
        _ARCHITECTURES[n] = arch
    return arch


def unregister_architecture(name: str) -> None:
    arch = _ARCHITECTURES.get(name)
    if arch is None:
        return
    for n in arch.names:
        _ARCHITECTURES.pop(n, None)


def known_architectures() -> List[str]:
    return sorted(_ARCHITECTURES)


def lookup_architecture(raw: Dict[str, Any]) -> Architecture:
    _ensure_builtin()
    keys = []
    archs = raw.get("architectures")
    if isinstance(archs, list) and archs:
        keys.append(str(archs[0]))
    if raw.get("model_type") is not None:
        keys.append(str(raw["model_type"]))
    if not keys:
        raise ConfigError("config.json: neither 'architectures' nor 'model_type' is given")
    for k in keys:
        if k in _ARCHITECTURES:
            return _ARCHITECTURES[k]
    raise ConfigError(f"Unsupported model_type: {' / '.join(keys)} "
                      f"(known: {', '.join(known_architectures())})")


def config_from_json(raw: Dict[str, Any]) -> ModelConfig:
    return lookup_architecture(raw).config_cls.from_json(raw)


def load_config(model_dir: str) -> ModelConfig:
    return config_from_json(read_config_json(model_dir))


def describe_model(cfg: ModelConfig):
    return lookup_architecture(cfg.raw).describe(cfg)


_builtin_done = False


def _ensure_builtin() -> None:
    global _builtin_done
    if not _builtin_done:
        _builtin_done = True
        from .. import models
        models.register_builtin()
