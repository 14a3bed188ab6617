from .base import (ConfigError, ModelConfig, config_from_dict, known_architectures, load_config,
                   lookup_architecture, register_architecture, save_config)
from .llama import LlamaConfig, RopeScaling
