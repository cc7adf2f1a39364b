"""The optimizer under the backward pass: a unit is updated as soon as the backward pass has left it.  On CPU the
update runs in place inside the backward pass, which checks the one thing the schedule assumes: every gradient of a
unit has been produced by then."""
import torch

from ksa_b200.config import get_preset
from ksa_b200.models import get_model_class
from ksa_b200.training.activations import set_activation_checkpointing
from ksa_b200.training.engine import TrainEngine


def _cfg(**over):
    return get_preset("qwen3-ksa-tiny").merge({"num_layers": 3, "summary_layer_freq": [1, 0, 1], "embed_dim": 64,
                                               "intermediate_dim": 128, "vocab_size": 256, "head_dim": 16, **over})


def _engine(overlap, accum=1, checkpointing=False, offload=False, **over):
    cfg = _cfg(**over)
    model = get_model_class(cfg.model_class)(cfg)
    model.init_weights(seed=0)
    if checkpointing:
        assert set_activation_checkpointing(model, model.get_checkpointable_module_classes()) == 3
    eng = TrainEngine(model, lr=1e-2, weight_decay=0.1, clip_value=1.0, grad_accum_steps=accum,
                      overlap_optimizer=overlap, cpu_offload=offload)
    return eng, cfg


def _train(eng, cfg, micro_steps, seed=3):
    g = torch.Generator().manual_seed(seed)
    out = []
    for _ in range(micro_steps):
        t = torch.randint(0, cfg.vocab_size, (2, 129), generator=g)
        out.append(float(eng.train_step(t[:, :-1].contiguous(), t[:, 1:].contiguous())))
    return out


def _same(e0, e1):
    for a, b in zip(e0.units, e1.units):
        assert torch.equal(a.master, b.master), a.name
        assert torch.equal(a.exp_avg, b.exp_avg) and torch.equal(a.exp_avg_sq, b.exp_avg_sq), a.name
        assert torch.equal(a.compute, b.compute), a.name


def test_units_are_updated_inside_the_backward_pass_and_training_is_bit_identical():
    e0, cfg = _engine(False)
    e1, _ = _engine(True)
    assert not e0.overlap_optimizer and e1.overlap_optimizer
    seen = []
    plain = e1._reduce_and_update
    e1._reduce_and_update = lambda u: (seen.append((u.name, e1._hooks_active)), plain(u))[1]
    l0, l1 = _train(e0, cfg, 3), _train(e1, cfg, 3)
    assert l0 == l1
    _same(e0, e1)
    assert float(e0.grad_norm()) == float(e1.grad_norm())
    # per step: head and the layers (last first) during the backward pass, the embedding unit after it
    assert [n for n, _ in seen[:5]] == ["head", "layer2", "layer1", "layer0", "embed"]
    assert [inside for _, inside in seen[:5]] == [True, True, True, True, False]
    assert len(seen) == 15 and e1.step_count == 3


def test_accumulation_windows_update_only_on_the_last_micro_step():
    e0, cfg = _engine(False, accum=2)
    e1, _ = _engine(True, accum=2)
    calls = []
    plain = e1._reduce_and_update
    e1._reduce_and_update = lambda u: (calls.append(e1.micro_step), plain(u))[1]
    assert _train(e0, cfg, 4) == _train(e1, cfg, 4)
    _same(e0, e1)
    # never during the first micro-step (micro_step 0); 1 = inside the second backward pass, 2 = after it (embedding)
    assert e1.step_count == 2 and calls.count(1) == 8 and calls.count(2) == 2 and len(calls) == 10


def test_with_activation_checkpointing_tied_weights_and_offloaded_state():
    for kw in (dict(checkpointing=True), dict(tie_word_embeddings=True), dict(offload=True)):
        e0, cfg = _engine(False, **kw)
        e1, _ = _engine(True, **kw)
        assert _train(e0, cfg, 2) == _train(e1, cfg, 2), kw
        e0.sync_state(); e1.sync_state()
        _same(e0, e1)


def test_an_optimizer_step_without_the_engines_backward_updates_everything():
    e1, cfg = _engine(True)
    e0, _ = _engine(False)
    for e in (e0, e1):
        for u in e.units:
            u.grad.copy_(torch.randn(u.grad.shape, generator=torch.Generator().manual_seed(5)) * 0.1)
            for s in u.slots:
                s.param._grad_written = True
        e._write_hyper()
        e.optimizer_step()
    _same(e0, e1)
