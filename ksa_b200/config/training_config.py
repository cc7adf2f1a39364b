"""Typed training configuration tree (``muse/config/training_config.py:62-281``,
``muse/config/dataset_config.py:51-116``) and the helpers that build it from a file, from parsed command-line
arguments, or from a checkpoint directory (``muse/config/utils.py:60-312``).

The recipe takes plain command-line flags, exactly like the reference's; :func:`training_config_from_args` gives the
same run as one validated object, which is what gets stored next to a checkpoint.
"""
from __future__ import annotations

import argparse
import json
import os
from typing import Any, Dict, Literal, Optional, Tuple

import yaml
from pydantic import Field, model_validator

from .base import BaseConfig, load_config, register_config


@register_config
class OptimizerConfig(BaseConfig):
    learning_rate: float = Field(default=1e-4, gt=0.0)
    weight_decay: float = Field(default=0.1, ge=0.0)
    beta1: float = Field(default=0.9, ge=0.0, lt=1.0)
    beta2: float = Field(default=0.95, ge=0.0, lt=1.0)
    eps: float = Field(default=1e-8, gt=0.0)


@register_config
class SchedulerConfig(BaseConfig):
    lr_scheduler_type: Literal["cosine", "cosine_v2", "wsd", "constant"] = "cosine"
    num_warmup_steps: int = Field(default=0, ge=0)
    num_decay_steps: int = Field(default=0, ge=0)
    num_training_steps: int = Field(default=1000, ge=1)
    num_epochs: int = Field(default=1, ge=1)
    min_lr: float = Field(default=0.0, ge=0.0)

    @model_validator(mode="after")
    def _steps(self):
        if self.num_warmup_steps >= self.num_training_steps:
            raise ValueError(f"num_warmup_steps ({self.num_warmup_steps}) must be less than num_training_steps "
                             f"({self.num_training_steps})")
        return self


@register_config
class CheckpointConfig(BaseConfig):
    output_dir: str
    save_checkpoint_per_step: int = Field(default=0, ge=0)
    save_checkpoint_every_epoch: bool = False
    resume_from: Optional[str] = None           # checkpoint directory
    resume_from_tag: Optional[str] = None       # ``global_step{N}``; default: the ``latest`` file
    resume_weights: bool = True
    resume_optimizer: bool = True
    resume_dataloader: bool = False
    load_weights_only: bool = False
    auto_resume_local_latest: bool = False
    enable_dataset_checkpointing: bool = False


@register_config
class LoggingConfig(BaseConfig):
    logging_per_step: int = Field(default=1, ge=1)
    monitor_datasource_loss: bool = False
    monitor_datasource_cnt: bool = False
    log_attn_stats: bool = False
    comment: Optional[str] = None
    commit_id: Optional[str] = None
    heartbeat_monitor: bool = False
    enable_profile: bool = False


@register_config
class DatasetConfig(BaseConfig):
    dataset_class: str = "KaiMMapDataset"
    dataset_config: Optional[str] = None        # path of the dataset JSON
    max_length: Optional[int] = Field(default=None, ge=1)
    batch_size: Optional[int] = Field(default=None, ge=1)
    num_workers: int = Field(default=0, ge=0)
    shuffle_buffer_size: int = Field(default=0, ge=0)
    use_dataset_load_balance: bool = False
    packing: bool = False
    extra_config: Dict[str, Any] = Field(default_factory=dict)


@register_config
class ParallelConfig(BaseConfig):
    context_parallel_size: int = Field(default=1, ge=1)
    fp32_weight: bool = True
    fp32_reduce: bool = True
    reshard_after_forward: bool = False
    cpu_offload: bool = False
    comm: Literal["fused", "collective"] = "fused"
    overlap: Literal["stream", "gemm"] = "stream"


@register_config
class TrainingConfig(BaseConfig):
    optimizer: OptimizerConfig = Field(default_factory=OptimizerConfig)
    scheduler: SchedulerConfig = Field(default_factory=SchedulerConfig)
    checkpoint: CheckpointConfig
    logging: LoggingConfig = Field(default_factory=LoggingConfig)
    dataset: DatasetConfig = Field(default_factory=DatasetConfig)
    parallel: ParallelConfig = Field(default_factory=ParallelConfig)
    model_config_path: Optional[str] = None
    model_dtype: Literal["bfloat16", "float16", "float32"] = "bfloat16"
    gradient_accumulation_steps: int = Field(default=1, ge=1)
    clip_range: float = Field(default=1.0, gt=0.0)
    enable_gradient_checkpointing: bool = False
    chunked_loss_minibatch_size: int = Field(default=2048, ge=1)
    disable_chunked_loss: bool = False
    freeze_llm: bool = False
    seed: int = 123


# ------------------------------------------------------------------------------ helpers
def load_config_from_file(path: str) -> Dict[str, Any]:
    """JSON or YAML file -> plain dict."""
    with open(path, "r", encoding="utf-8") as f:
        return yaml.safe_load(f) if path.endswith((".yml", ".yaml")) else json.load(f)


def merge_configs(base: Dict[str, Any], override: Dict[str, Any]) -> Dict[str, Any]:
    """Recursive dict merge; ``None`` values of ``override`` do not erase anything."""
    out = dict(base)
    for k, v in override.items():
        if isinstance(v, dict) and isinstance(out.get(k), dict):
            out[k] = merge_configs(out[k], v)
        elif v is not None:
            out[k] = v
    return out


_ARG_MAP: Dict[str, Tuple[str, str]] = {
    "learning_rate": ("optimizer", "learning_rate"), "weight_decay": ("optimizer", "weight_decay"),
    "beta1": ("optimizer", "beta1"), "beta2": ("optimizer", "beta2"),
    "lr_scheduler_type": ("scheduler", "lr_scheduler_type"), "num_warmup_steps": ("scheduler", "num_warmup_steps"),
    "num_decay_steps": ("scheduler", "num_decay_steps"), "num_training_steps": ("scheduler", "num_training_steps"),
    "num_epochs": ("scheduler", "num_epochs"), "min_lr": ("scheduler", "min_lr"),
    "output_dir": ("checkpoint", "output_dir"), "save_checkpoint_per_step": ("checkpoint", "save_checkpoint_per_step"),
    "save_checkpoint_every_epoch": ("checkpoint", "save_checkpoint_every_epoch"),
    "checkpoint_dir": ("checkpoint", "resume_from"), "checkpoint_id": ("checkpoint", "resume_from_tag"),
    "resume_weights": ("checkpoint", "resume_weights"), "resume_optimizer": ("checkpoint", "resume_optimizer"),
    "resume_dataloader": ("checkpoint", "resume_dataloader"),
    "enable_dataset_checkpointing": ("checkpoint", "enable_dataset_checkpointing"),
    "logging_per_step": ("logging", "logging_per_step"), "monitor_datasource_loss": ("logging", "monitor_datasource_loss"),
    "log_attn_stats": ("logging", "log_attn_stats"), "comment": ("logging", "comment"),
    "commit_id": ("logging", "commit_id"), "enable_profile": ("logging", "enable_profile"),
    "dataset_class": ("dataset", "dataset_class"), "dataset_config": ("dataset", "dataset_config"),
    "max_length": ("dataset", "max_length"), "batch_size": ("dataset", "batch_size"),
    "shuffle_buffer_size": ("dataset", "shuffle_buffer_size"),
    "use_dataset_load_balance": ("dataset", "use_dataset_load_balance"), "packing": ("dataset", "packing"),
    "context_parallel_size": ("parallel", "context_parallel_size"), "fp32_weight": ("parallel", "fp32_weight"),
    "fp32_reduce": ("parallel", "fp32_reduce"), "reshard_after_forward": ("parallel", "reshard_after_forward"),
    "cpu_offload": ("parallel", "cpu_offload"), "comm": ("parallel", "comm"), "overlap": ("parallel", "overlap"),
}
_TOP_ARGS = {"model_config": "model_config_path", "model_dtype": "model_dtype",
             "gradient_accumulation_steps": "gradient_accumulation_steps", "clip_range": "clip_range",
             "enable_gradient_checkpointing": "enable_gradient_checkpointing",
             "chunked_loss_minibatch_size": "chunked_loss_minibatch_size", "disable_chunked_loss": "disable_chunked_loss",
             "seed": "seed"}


def load_config_from_args(args: argparse.Namespace) -> Dict[str, Any]:
    """Parsed recipe flags -> nested dict in the shape of :class:`TrainingConfig` (unset flags are left out)."""
    out: Dict[str, Any] = {}
    for name, value in vars(args).items():
        if value is None:
            continue
        if name in _ARG_MAP:
            group, key = _ARG_MAP[name]
            out.setdefault(group, {})[key] = value
        elif name in _TOP_ARGS:
            out[_TOP_ARGS[name]] = value
    return out


def training_config_from_args(args: argparse.Namespace, config_file: Optional[str] = None) -> TrainingConfig:
    """File values first, command-line flags on top."""
    base = load_config_from_file(config_file) if config_file else {}
    base.pop("__class__", None)
    return TrainingConfig(**merge_configs(base, load_config_from_args(args)))


def save_config_to_checkpoint(config: BaseConfig, checkpoint_dir: str, name: str = "training_config.json") -> str:
    os.makedirs(checkpoint_dir, exist_ok=True)
    path = os.path.join(checkpoint_dir, name)
    config.save(path)
    return path


def save_all_configs_to_checkpoint(checkpoint_dir: str, **configs: BaseConfig) -> Dict[str, str]:
    """``save_all_configs_to_checkpoint(dir, training=..., model=...)`` writes ``<name>_config.json`` files."""
    return {k: save_config_to_checkpoint(c, checkpoint_dir, f"{k}_config.json") for k, c in configs.items()}


def load_configs_from_checkpoint(checkpoint_dir: str) -> Dict[str, BaseConfig]:
    out: Dict[str, BaseConfig] = {}
    for fn in sorted(os.listdir(checkpoint_dir)):
        if fn.endswith("_config.json"):
            out[fn[: -len("_config.json")]] = load_config(os.path.join(checkpoint_dir, fn))
    return out
