"""Typed configurations, one class per architecture."""
from .base import ConfigError, ModelConfig, key, read_config_json
from .bolelix import BolelixConfig
from .lopazen import LopazenConfig
from .musavik import MusavikConfig
from .qwen3 import Qwen3Config
from .susalorn import SusalornConfig

__all__ = ["BolelixConfig", "ConfigError", "LopazenConfig", "ModelConfig", "MusavikConfig", "Qwen3Config", "SusalornConfig", "key", "read_config_json"]
