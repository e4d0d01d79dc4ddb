from .base import ConfigError, read_config_json
from .qwen2_moe import Qwen2MoeConfig

__all__ = ["ConfigError", "read_config_json", "Qwen2MoeConfig"]
