"""Model descriptions. Each built-in architecture is one module of this package that registers itself (its names,
its configuration class, its `describe`) when imported; `BUILTIN` lists them, and the registry imports them on its
first lookup. An architecture from outside the package calls `config.register_architecture` itself."""
import importlib

from .causal_lm import CausalLM

BUILTIN = ("minicpm4",)


def register_builtin() -> None:
    for name in BUILTIN:
        importlib.import_module(f"{__name__}.{name}")
