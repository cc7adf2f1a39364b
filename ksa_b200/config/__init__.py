from .base import BaseConfig, config_classes, load_config, register_config
from .model_config import (ModelConfig, Qwen3Config, Qwen3SummaryAttentionConfig, get_preset, parse_layer_pattern,
                           PRESETS)

__all__ = ["BaseConfig", "config_classes", "load_config", "register_config", "ModelConfig", "Qwen3Config",
           "Qwen3SummaryAttentionConfig", "get_preset", "parse_layer_pattern", "PRESETS"]
