from .model_config import (ConfigError, MiniCPM4Config, ModelConfig, RopeScaling, config_fields,
                           parse_dtype_name, read_config_json)
from .registry import (Architecture, config_from_json, describe_model, known_architectures, load_config,
                       lookup_architecture, register_architecture, unregister_architecture)
