"""Typed training configuration: flags + file merge, validation, checkpoint round trip."""
import argparse
import json

import pytest
from pydantic import ValidationError

from ksa_b200.config import (TrainingConfig, load_configs_from_checkpoint, merge_configs, get_preset,
                             save_all_configs_to_checkpoint, training_config_from_args)


def test_flags_override_file_and_validate(tmp_path):
    f = tmp_path / "train.json"
    f.write_text(json.dumps({"checkpoint": {"output_dir": "out", "save_checkpoint_per_step": 50},
                             "optimizer": {"learning_rate": 3e-4}, "seed": 7}))
    args = argparse.Namespace(learning_rate=1e-5, num_training_steps=1600, num_warmup_steps=10, lr_scheduler_type="wsd",
                              context_parallel_size=8, output_dir=None, comment="c", commit_id="abc", seed=None,
                              unrelated_flag=3)
    cfg = training_config_from_args(args, str(f))
    assert cfg.optimizer.learning_rate == 1e-5 and cfg.checkpoint.output_dir == "out"
    assert cfg.checkpoint.save_checkpoint_per_step == 50 and cfg.seed == 7
    assert cfg.scheduler.lr_scheduler_type == "wsd" and cfg.parallel.context_parallel_size == 8
    with pytest.raises(ValidationError):
        TrainingConfig(checkpoint={"output_dir": "o"}, scheduler={"num_warmup_steps": 10, "num_training_steps": 5})
    with pytest.raises(ValidationError):
        TrainingConfig(checkpoint={"output_dir": "o"}, not_a_field=1)
    with pytest.raises(ValidationError):
        cfg.clip_range = -1.0            # assignments are validated too


def test_merge_and_checkpoint_round_trip(tmp_path):
    assert merge_configs({"a": {"b": 1, "c": 2}, "d": 3}, {"a": {"b": 5}, "d": None}) == {"a": {"b": 5, "c": 2}, "d": 3}
    cfg = TrainingConfig(checkpoint={"output_dir": str(tmp_path)})
    save_all_configs_to_checkpoint(str(tmp_path), training=cfg, model=get_preset("qwen3-ksa-tiny"))
    back = load_configs_from_checkpoint(str(tmp_path))
    assert back["training"] == cfg and back["model"] == get_preset("qwen3-ksa-tiny")
