"""Checkpoint round trip (DCP layout, latest file, selective resume) and DCP -> HF conversion on CPU."""
import json
import os

import torch

from ksa_b200.config import get_preset
from ksa_b200.models import get_model_class
from ksa_b200.training.checkpoint import (AppState, DistributedCheckpointer, dcp_to_state_dict, get_checkpoint_path,
                                          load_checkpoint, save_checkpoint)
from ksa_b200.training.common import StepScheduler
from ksa_b200.training.engine import TrainEngine
from ksa_b200.tools.convert import convert_dcp_to_hf, flatten_model_state, hf_config_from_model_config


def _engine(seed=0):
    cfg = get_preset("qwen3-ksa-tiny").merge({"num_layers": 2, "summary_layer_freq": [1, 0], "embed_dim": 64,
                                               "intermediate_dim": 128, "vocab_size": 256, "head_dim": 16})
    model = get_model_class(cfg.model_class)(cfg)
    model.init_weights(seed=seed)
    return TrainEngine(model, lr=1e-2, weight_decay=0.1), cfg


def _train(eng, cfg, steps, seed=3):
    g = torch.Generator().manual_seed(seed)
    for _ in range(steps):
        t = torch.randint(0, cfg.vocab_size, (1, 129), generator=g)
        eng.train_step(t[:, :-1].contiguous(), t[:, 1:].contiguous())


def test_save_resume_bitwise_and_layout(tmp_path):
    eng, cfg = _engine()
    sched = StepScheduler(1, 10, 2)
    _train(eng, cfg, 2)
    sched.step(); sched.step()
    ck = DistributedCheckpointer()
    path = save_checkpoint(AppState(eng, sched), ck, str(tmp_path), 2)
    assert os.path.basename(path) == "global_step2" and (tmp_path / "latest").read_text() == "global_step2"
    assert get_checkpoint_path(str(tmp_path)) == path and get_checkpoint_path(str(tmp_path), "2") == path
    tree = flatten_model_state(dcp_to_state_dict(path))
    assert "model.layers.0.attn.q_proj_summary.weight" in tree and "model.layers.1.mlp.w3.weight" in tree
    assert "summary_embedding.weight" in tree and "model.output.weight" in tree
    # resume into a differently initialised engine, continue, and compare with uninterrupted training
    eng2, _ = _engine(seed=5)
    sched2 = StepScheduler(1, 10, 2)
    step = load_checkpoint(AppState(eng2, sched2), ck, str(tmp_path))
    assert step == 2 and sched2.global_step == 2 and eng2.step_count == 2
    _train(eng, cfg, 2, seed=9)
    _train(eng2, cfg, 2, seed=9)
    for a, b in zip(eng.units, eng2.units):
        assert torch.equal(a.master, b.master) and torch.equal(a.exp_avg_sq, b.exp_avg_sq)


def test_resume_weights_only(tmp_path):
    eng, cfg = _engine()
    _train(eng, cfg, 1)
    ck = DistributedCheckpointer()
    save_checkpoint(AppState(eng), ck, str(tmp_path), 1)
    eng2, _ = _engine(seed=7)
    load_checkpoint(AppState(eng2, skip_optimizer=True, skip_training_state=True), ck, str(tmp_path))
    assert eng2.step_count == 0
    for a, b in zip(eng.units, eng2.units):
        assert torch.equal(a.master, b.master) and b.exp_avg.abs().sum() == 0


def test_convert_dcp_to_hf(tmp_path):
    from safetensors.torch import load_file
    eng, cfg = _engine()
    ck = DistributedCheckpointer()
    save_checkpoint(AppState(eng), ck, str(tmp_path), 7)
    template = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "ksa_b200", "hf")
    out = convert_dcp_to_hf(str(tmp_path), "global_step7", template, dtype="fp32", remap="muse2hf",
                            config_overrides=hf_config_from_model_config(cfg))
    files = os.listdir(out)
    assert "config.json" in files and any(f.endswith(".safetensors") for f in files)
    hf = {}
    for f in files:
        if f.endswith(".safetensors"):
            hf.update(load_file(os.path.join(out, f)))
    assert hf["model.embed_tokens.weight"].shape[0] == cfg.vocab_size + cfg.summary_token_num
    assert hf["lm_head.weight"].shape[0] == cfg.vocab_size + cfg.summary_token_num
    assert json.load(open(os.path.join(out, "config.json")))["vocab_size"] == cfg.vocab_size + cfg.summary_token_num
    model = get_model_class(cfg.model_class)(cfg)
    model.load_state_dict(model.convert_hf_state_dict(hf))
    for (n, a), (_, b) in zip(model.state_dict().items(), eng.model.state_dict().items()):
        assert torch.allclose(a, b.float()), n


def test_dcp2torch_single_file_and_safetensors(tmp_path):
    """``python -m ksa_b200.tools.dcp2torch``: a checkpoint becomes one ``torch.save`` file (model only, or everything)
    or sharded safetensors, with the parameter names (the reference's) and values of the model that was saved."""
    from safetensors.torch import load_file
    from ksa_b200.tools import dcp2torch
    eng, cfg = _engine()
    _train(eng, cfg, 2)
    save_checkpoint(AppState(eng), DistributedCheckpointer(), str(tmp_path), 2)
    dcp = get_checkpoint_path(str(tmp_path), 2) if callable(get_checkpoint_path) else os.path.join(str(tmp_path), "global_step2")
    want = {k: v.detach() for k, v in eng.model.muse_state_dict().items()}    # checkpoints use the reference's names
    # one file, model only
    dcp2torch.main([dcp, str(tmp_path / "model.pt")])
    got = torch.load(str(tmp_path / "model.pt"), weights_only=True)
    assert set(got) == set(want)
    for k in want:
        assert torch.equal(got[k].to(want[k].dtype), want[k]), k
    # one file, everything: optimizer and training state travel too
    dcp2torch.main([dcp, str(tmp_path / "all.pt"), "--all"])
    everything = torch.load(str(tmp_path / "all.pt"), weights_only=False)
    flat = json.dumps(sorted(str(k) for k in everything))
    assert "app" in flat
    # sharded safetensors into a directory
    dcp2torch.main([dcp, str(tmp_path / "st"), "--safetensors"])
    files = [f for f in os.listdir(tmp_path / "st") if f.endswith(".safetensors")]
    assert files
    loaded = {}
    for f in files:
        loaded.update(load_file(str(tmp_path / "st" / f)))
    assert set(loaded) == set(want)
    for k in want:
        assert torch.equal(loaded[k].to(want[k].dtype), want[k]), k


def test_training_state_keys_can_be_skipped_required_and_extended(tmp_path):
    """Entries of the training state are restored one by one: named ones can be left out, others demanded, and
    further objects or values ride along under their own names."""
    import pytest

    class Counter:
        def __init__(self, n=0):
            self.n = n

        def state_dict(self):
            return {"n": self.n}

        def load_state_dict(self, s):
            self.n = s["n"]
    eng, cfg = _engine()
    sched = StepScheduler(1, 10, 2)
    _train(eng, cfg, 2)
    sched.step(); sched.step()
    ck = DistributedCheckpointer()
    save_checkpoint(AppState(eng, sched, extra_training_state={"tokens_seen": Counter(4096), "note": "stage 8k"}),
                    ck, str(tmp_path), 2)
    # everything back, extras included
    eng2, _ = _engine(seed=5)
    sched2, extra = StepScheduler(1, 10, 2), {"tokens_seen": Counter(), "note": ""}   # the loader names what it wants
    load_checkpoint(AppState(eng2, sched2, extra_training_state=extra,
                             required_training_state_keys=["step_scheduler", "tokens_seen"]), ck, str(tmp_path))
    assert sched2.global_step == 2 and extra["tokens_seen"].n == 4096 and extra["note"] == "stage 8k"
    # the step scheduler and one extra are left alone
    eng3, _ = _engine(seed=5)
    sched3, extra3 = StepScheduler(1, 10, 2), {"tokens_seen": Counter(7)}
    load_checkpoint(AppState(eng3, sched3, extra_training_state=extra3,
                             skip_training_state_keys=["step_scheduler", "tokens_seen"]), ck, str(tmp_path))
    assert sched3.global_step == 0 and extra3["tokens_seen"].n == 7 and eng3.step_count == 2
    # a demanded entry that the checkpoint lacks
    eng4, _ = _engine(seed=5)
    with pytest.raises(Exception, match="Missing required training state keys"):
        load_checkpoint(AppState(eng4, required_training_state_keys=["ema"]), ck, str(tmp_path))


def test_frozen_parameters_are_neither_decayed_nor_updated_and_survive_a_checkpoint(tmp_path):
    """Distillation freezes the base weights before the engine is built: they stay out of the optimizer units, so
    weight decay leaves them bit-identical, while the summary parameters train; a checkpoint carries both."""
    from ksa_b200.training.common import freeze_params_by_pattern
    cfg = get_preset("qwen3-ksa-tiny").merge({"num_layers": 2, "summary_layer_freq": [1, 0], "embed_dim": 64,
                                               "intermediate_dim": 128, "vocab_size": 256, "head_dim": 16})
    model = get_model_class(cfg.model_class)(cfg)
    model.init_weights(seed=0)
    stats = freeze_params_by_pattern(model, ["summary_embedding", "_summary"])
    assert stats["trainable"] > 0 and stats["frozen"] > 0
    eng = TrainEngine(model, lr=1e-2, weight_decay=0.5)
    before = {n: p.detach().clone() for n, p in model.named_parameters()}
    _train(eng, cfg, 3)
    changed = 0
    for n, p in model.named_parameters():
        if p.requires_grad:
            changed += int(not torch.equal(p.detach(), before[n]))
        else:
            assert torch.equal(p.detach(), before[n]), f"frozen parameter {n} changed"
    assert changed > 0
    assert {s.name for u in eng.units for s in u.slots}.isdisjoint(s.name for s in eng.frozen_slots)
    ck = DistributedCheckpointer()
    path = save_checkpoint(AppState(eng), ck, str(tmp_path), 3)
    tree = flatten_model_state(dcp_to_state_dict(path))
    assert "model.layers.0.attn.q_proj.weight" in tree and "model.layers.0.attn.q_proj_summary.weight" in tree
    model2 = get_model_class(cfg.model_class)(cfg)
    model2.init_weights(seed=4)
    freeze_params_by_pattern(model2, ["summary_embedding", "_summary"])
    eng2 = TrainEngine(model2, lr=1e-2, weight_decay=0.5)
    load_checkpoint(AppState(eng2), ck, str(tmp_path))
    for (n, a), (_, b) in zip(model.named_parameters(), model2.named_parameters()):
        assert torch.equal(a.detach(), b.detach()), n
