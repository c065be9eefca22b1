from .model_config import ConfigError, ModelConfig, RopeScaling, config_fields, parse_dtype_name, read_config_json
from .registry import (Architecture, config_from_json, describe_model, known_architectures, load_config,
                       lookup_architecture, register_architecture, unregister_architecture)


def __getattr__(name):
    # configuration classes of the built-in architectures live beside their models
    if name == "MiniCPM4Config":
        from ..models.minicpm4 import MiniCPM4Config
        return MiniCPM4Config
    raise AttributeError(name)
