"""The model on the sm_100a kernels against the same model in fp32 on the CPU formulas; engine behaviour."""
import copy

import pytest
import torch

from ksa_b200.config import get_preset
from ksa_b200.models import get_model_class
from ksa_b200.ops import _lib
from ksa_b200.training.engine import TrainEngine

pytestmark = pytest.mark.gpu


def _tiny(head_dim=64, chunk=64, **over):
    cfg = get_preset("qwen3-ksa-tiny")
    return cfg.merge({"head_dim": head_dim, "summary_chunk_size": chunk, **over})


@pytest.mark.parametrize("head_dim,chunk", [(64, 64), (128, 128)])
def test_logits_and_loss_match_fp32_cpu(head_dim, chunk):
    cfg = _tiny(head_dim, chunk)
    torch.manual_seed(0)
    ref_model = get_model_class(cfg.model_class)(cfg)
    ref_model.init_weights(seed=0)
    # round the weights to bf16 once so that both sides start from identical values
    with torch.no_grad():
        for p in ref_model.parameters():
            p.copy_(p.to(torch.bfloat16).float())
    gpu_model = copy.deepcopy(ref_model).to("cuda").to(torch.bfloat16)
    tokens = torch.randint(0, cfg.vocab_size, (2, 1024))
    labels = torch.roll(tokens, -1, 1)
    labels[:, -1] = -100
    logits = gpu_model(tokens.cuda()).float().cpu()
    expect = ref_model(tokens)
    _lib.check_status()
    err = (logits - expect).norm() / expect.norm()
    assert err < 3e-2, err
    loss = gpu_model(tokens.cuda(), labels=labels.cuda())
    loss.backward()
    loss_ref = ref_model(tokens, labels=labels)
    loss_ref.backward()
    _lib.check_status()
    assert abs(loss.item() - loss_ref.item()) < 2e-2
    for (n, a), (_, b) in zip(gpu_model.named_parameters(), ref_model.named_parameters()):
        assert a.grad is not None, n
        e = (a.grad.float().cpu() - b.grad).norm() / b.grad.norm().clamp_min(1e-6)
        assert e < 8e-2, (n, e.item())


def test_engine_step_and_graph_replay_agree():
    cfg = _tiny(128, 128, embed_dim=512)
    torch.manual_seed(0)
    base = get_model_class(cfg.model_class)(cfg)
    base.init_weights(seed=0)
    tokens = torch.randint(0, cfg.vocab_size, (1, 2, 513), device="cuda").repeat(4, 1, 1)  # same batch 4 times
    results = []
    for graphed in (False, True):
        model = copy.deepcopy(base).to("cuda").to(torch.bfloat16)
        eng = TrainEngine(model, lr=1e-3, weight_decay=0.1, clip_value=1.0)
        fn = eng.graphed_step if graphed else eng.train_step
        losses = [float(fn(t[:, :-1].contiguous(), t[:, 1:].contiguous())) for t in tokens]
        _lib.check_status()
        results.append((losses, [u.master.clone() for u in eng.units], float(eng.grad_norm())))
    (l0, m0, g0), (l1, m1, g1) = results
    assert l0[-1] < l0[0]
    assert all(abs(a - b) < 2e-2 for a, b in zip(l0, l1)), (l0, l1)
    assert abs(g0 - g1) < 0.05 * g0
    for a, b in zip(m0, m1):
        assert (a - b).norm() <= 2e-2 * a.norm()


def test_grad_accumulation_equals_large_batch():
    cfg = _tiny(64, 64)
    torch.manual_seed(0)
    base = get_model_class(cfg.model_class)(cfg)
    base.init_weights(seed=0)
    toks = torch.randint(0, cfg.vocab_size, (2, 1, 513), device="cuda")
    m1 = copy.deepcopy(base).to("cuda").to(torch.bfloat16)
    e1 = TrainEngine(m1, lr=1e-3, grad_accum_steps=2)
    for t in toks:
        e1.train_step(t[:, :-1].contiguous(), t[:, 1:].contiguous())
    m2 = copy.deepcopy(base).to("cuda").to(torch.bfloat16)
    e2 = TrainEngine(m2, lr=1e-3)
    both = toks.reshape(2, 513)
    e2.train_step(both[:, :-1].contiguous(), both[:, 1:].contiguous())
    _lib.check_status()
    assert e1.step_count == 1 and e2.step_count == 1
    for a, b in zip(e1.units, e2.units):
        assert (a.master - b.master).norm() <= 3e-3 * b.master.norm()


def test_optimizer_state_offloaded_to_pinned_host_memory_matches_resident_state():
    """Master weights and moments in pinned host memory, updated through the two-slot staging ring: identical
    gradients give bit-identical state, and a few real steps stay within the run-to-run noise of the backward."""
    cfg = _tiny(64, 64)
    torch.manual_seed(0)
    base = get_model_class(cfg.model_class)(cfg)
    base.init_weights(seed=0)
    engines = []
    for offload in (False, True):
        model = copy.deepcopy(base).to("cuda").to(torch.bfloat16)
        engines.append(TrainEngine(model, lr=1e-3, weight_decay=0.1, clip_value=1.0, cpu_offload=offload))
    e0, e1 = engines
    assert all(u.master.is_pinned() and u.master.device.type == "cpu" for u in e1.units)
    g = torch.Generator(device="cuda").manual_seed(5)
    for step in range(3):                                    # the optimizer alone, on the same gradients
        for a, b in zip(e0.units, e1.units):
            a.grad.copy_(torch.randn(a.grad.shape, device="cuda", generator=g) * 0.05)
            b.grad.copy_(a.grad)
        for e in engines:
            for u in e.units:
                for s in u.slots:
                    s.param._grad_written = True
            e._write_hyper()
            e.optimizer_step()
            e.step_count += 1
    e1.sync_state()
    _lib.check_status()
    for a, b in zip(e0.units, e1.units):
        assert torch.equal(a.master.cpu(), b.master) and torch.equal(a.exp_avg.cpu(), b.exp_avg)
        assert torch.equal(a.exp_avg_sq.cpu(), b.exp_avg_sq) and torch.equal(a.compute, b.compute)
    toks = torch.randint(0, cfg.vocab_size, (3, 2, 513), device="cuda")
    l0 = [float(e0.train_step(t[:, :-1].contiguous(), t[:, 1:].contiguous())) for t in toks]
    l1 = [float(e1.graphed_step(t[:, :-1].contiguous(), t[:, 1:].contiguous())) for t in toks]   # falls back to eager
    e1.sync_state()
    _lib.check_status()
    assert all(abs(a - b) < 2e-2 for a, b in zip(l0, l1)), (l0, l1)
    for a, b in zip(e0.units, e1.units):
        assert (a.master.cpu() - b.master).norm() <= 2e-2 * b.master.norm()
    n = sum(u.host_state.numel() for u in e1.units) * 4
    assert e1._offload.h2d_bytes == 6 * n and e1._offload.d2h_bytes == 6 * n


def test_deterministic_mode_makes_training_steps_bit_reproducible():
    """``ops.set_deterministic(True)``: two runs of the same three steps give bit-identical master weights, moments,
    losses and gradient norms (the attention backward, QK-norm weight gradients, embedding gradient and the sum of
    squared gradients all sum in a fixed order), and stay close to the default mode."""
    from ksa_b200 import ops
    cfg = _tiny(128, 128, embed_dim=512)
    torch.manual_seed(0)
    base = get_model_class(cfg.model_class)(cfg)
    base.init_weights(seed=0)
    toks = torch.randint(0, cfg.vocab_size, (3, 2, 513), device="cuda")
    toks[:, :, 100:140] = 7                      # one id many times: its embedding row collects many gradient rows

    def run():
        model = copy.deepcopy(base).to("cuda").to(torch.bfloat16)
        eng = TrainEngine(model, lr=1e-3, weight_decay=0.1, clip_value=1.0)
        out = []
        for t in toks:
            loss = eng.train_step(t[:, :-1].contiguous(), t[:, 1:].contiguous())
            out.append((float(loss), float(eng.grad_norm())))
        _lib.check_status()
        return out, [(u.master.clone(), u.exp_avg_sq.clone()) for u in eng.units]

    free = run()
    ops.set_deterministic(True)
    try:
        a, b = run(), run()
    finally:
        ops.set_deterministic(False)
    assert a[0] == b[0], (a[0], b[0])
    for (m0, v0), (m1, v1) in zip(a[1], b[1]):
        assert torch.equal(m0, m1) and torch.equal(v0, v1)
    for (l0, g0), (l1, g1) in zip(a[0], free[0]):
        assert abs(l0 - l1) < 2e-2 and abs(g0 - g1) < 0.05 * g1
    for (m0, _), (m1, _) in zip(a[1], free[1]):
        assert (m0 - m1).norm() <= 2e-2 * m1.norm()


def test_optimizer_under_the_backward_pass_matches_the_optimizer_after_it():
    """Units updated on a side stream while the backward pass still runs against the whole optimizer after the
    backward pass: bit for bit with deterministic kernels (eager), within run-to-run noise when the overlapped step
    is replayed from a CUDA graph."""
    from ksa_b200 import ops
    cfg = _tiny(128, 128, embed_dim=512)
    torch.manual_seed(0)
    base = get_model_class(cfg.model_class)(cfg)
    base.init_weights(seed=0)
    toks = torch.randint(0, cfg.vocab_size, (4, 2, 513), device="cuda")

    def run(overlap, graphed):
        model = copy.deepcopy(base).to("cuda").to(torch.bfloat16)
        eng = TrainEngine(model, lr=1e-3, weight_decay=0.1, clip_value=1.0, overlap_optimizer=overlap)
        assert eng.overlap_optimizer == overlap
        fn = eng.graphed_step if graphed else eng.train_step
        losses = [float(fn(t[:, :-1].contiguous(), t[:, 1:].contiguous())) for t in toks]
        torch.cuda.synchronize()
        _lib.check_status()
        assert bool(eng._graphs) == (graphed and not ops.is_deterministic())
        return losses, float(eng.grad_norm()), [(u.master.clone(), u.exp_avg.clone(), u.compute.clone())
                                                for u in eng.units]

    ops.set_deterministic(True)
    try:
        ref_run, got = run(False, False), run(True, False)
        assert run(True, True)[0] == ref_run[0]          # deterministic mode keeps the graph entry point eager
    finally:
        ops.set_deterministic(False)
    assert got[0] == ref_run[0] and got[1] == ref_run[1], (got[0], ref_run[0])
    for a, b in zip(got[2], ref_run[2]):
        assert all(torch.equal(x, y) for x, y in zip(a, b))
    replayed = run(True, True)
    assert all(abs(a - b) < 2e-2 for a, b in zip(replayed[0], ref_run[0])), (replayed[0], ref_run[0])
    for a, b in zip(replayed[2], ref_run[2]):
        assert (a[0] - b[0]).norm() <= 2e-2 * b[0].norm()
