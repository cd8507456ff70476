from .model_config import ConfigError, GqaMtpConfig, read_config_json, write_config_json, UPSTREAM_ALIASES
from .engine_config import EngineConfig

__all__ = ["ConfigError", "GqaMtpConfig", "EngineConfig", "read_config_json", "write_config_json",
           "UPSTREAM_ALIASES"]
