from .base import ConfigError, ModelConfig, field, read_config_json, architecture_name
from .gpt2 import GPT2Config

__all__ = ["ConfigError", "ModelConfig", "field", "read_config_json", "architecture_name", "GPT2Config"]
