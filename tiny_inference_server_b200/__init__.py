"""A small, whole, single-GPU inference engine for B200 (sm_100a): the GQA decoder with
multi-token-prediction heads, from a model folder to generated tokens."""
from .config import ConfigError, EngineConfig, GqaMtpConfig
from .registry import (architectures, build_model, config_from_dict, config_from_folder, register_architecture,
                       register_part)

__all__ = ["ConfigError", "EngineConfig", "GqaMtpConfig", "architectures", "build_model", "config_from_dict",
           "config_from_folder", "register_architecture", "register_part"]
__version__ = "0.1.0"
