from .base import ConfigError, ModelConfig, parse_config_json, read_config_json
from .llama import LlamaConfig, RopeScaling

__all__ = ["ConfigError", "ModelConfig", "LlamaConfig", "RopeScaling",
           "parse_config_json", "read_config_json"]
