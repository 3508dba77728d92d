from .model_config import (ConfigError, LlamaConfig, RopeScaling, config_from_json_dict, known_architectures,
                           load_config, register_config_class, save_config)
from .registry import MODEL_CONFIGS, get_config, register_config

__all__ = ["ConfigError", "LlamaConfig", "RopeScaling", "config_from_json_dict", "known_architectures",
           "load_config", "register_config_class", "save_config", "MODEL_CONFIGS", "get_config", "register_config"]
