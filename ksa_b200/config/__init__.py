from .base import BaseConfig, config_classes, load_config, register_config
from .model_config import (ModelConfig, Qwen3Config, Qwen3SummaryAttentionConfig, get_preset, parse_layer_pattern,
                           PRESETS)

from .training_config import (CheckpointConfig, DatasetConfig, LoggingConfig, OptimizerConfig, ParallelConfig,
                              SchedulerConfig, TrainingConfig, load_config_from_args, load_config_from_file,
                              load_configs_from_checkpoint, merge_configs, save_all_configs_to_checkpoint,
                              save_config_to_checkpoint, training_config_from_args)

__all__ = ["CheckpointConfig", "DatasetConfig", "LoggingConfig", "OptimizerConfig", "ParallelConfig", "SchedulerConfig",
           "TrainingConfig", "load_config_from_args", "load_config_from_file", "load_configs_from_checkpoint",
           "merge_configs", "save_all_configs_to_checkpoint", "save_config_to_checkpoint", "training_config_from_args",
           "BaseConfig", "config_classes", "load_config", "register_config", "ModelConfig", "Qwen3Config",
           "Qwen3SummaryAttentionConfig", "get_preset", "parse_layer_pattern", "PRESETS"]
