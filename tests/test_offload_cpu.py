"""Optimizer state offloaded to host memory: the staging ring's bookkeeping, and training that is bit-identical to
training with the state on the device (single process, two gloo ranks, and across a checkpoint)."""
import os
import socket

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from ksa_b200.config import get_preset
from ksa_b200.models import get_model_class
from ksa_b200.training.checkpoint import AppState, DistributedCheckpointer, load_checkpoint, save_checkpoint
from ksa_b200.training.engine import TrainEngine
from ksa_b200.training.offload import OptimizerStateOffload, host_state


def _cfg():
    return get_preset("qwen3-ksa-tiny").merge({"num_layers": 3, "summary_layer_freq": [1, 0, 1], "embed_dim": 64,
                                               "intermediate_dim": 128, "vocab_size": 256, "head_dim": 16})


def _engine(offload, seed=0, **kw):
    cfg = _cfg()
    model = get_model_class(cfg.model_class)(cfg)
    model.init_weights(seed=seed)
    return TrainEngine(model, lr=1e-2, weight_decay=0.1, clip_value=1.0, cpu_offload=offload, **kw), cfg


def _train(eng, cfg, steps, seed=3):
    g = torch.Generator().manual_seed(seed)
    out = []
    for _ in range(steps):
        t = torch.randint(0, cfg.vocab_size, (1, 129), generator=g)
        out.append(float(eng.train_step(t[:, :-1].contiguous(), t[:, 1:].contiguous())))
    return out


def test_staging_ring_round_trip_and_slot_reuse():
    dev = torch.device("cpu")
    hosts = [host_state(n, dev) for n in (5, 8, 3, 8)]
    for i, h in enumerate(hosts):
        h.copy_(torch.arange(h.numel(), dtype=torch.float32).view_as(h) + 100 * i)
    ring = OptimizerStateOffload(dev, 8, slots=2)
    assert ring.staging.shape == (2, 3, 8)
    for idx in (3, 2, 1, 0):                       # the order of an optimizer step: last unit first
        m, a, b = ring.acquire(idx, hosts[idx])
        if idx > 0:
            ring.prefetch(idx - 1, hosts[idx - 1])   # the other slot: must not disturb the views in use
        assert torch.equal(m, hosts[idx][0]) and torch.equal(b, hosts[idx][2]) and m.numel() == hosts[idx].shape[1]
        m += 1.0
        b *= 2.0
        before = hosts[idx].clone()
        ring.release(idx, hosts[idx])
        assert torch.equal(hosts[idx][0], before[0] + 1.0) and torch.equal(hosts[idx][1], before[1])
        assert torch.equal(hosts[idx][2], before[2] * 2.0)
    # every unit went in and out once
    total = sum(h.numel() for h in hosts) * 4
    assert ring.h2d_bytes == total and ring.d2h_bytes == total
    # a unit whose host copy changed behind the ring's back is loaded afresh after synchronize()
    ring.prefetch(1, hosts[1])
    hosts[1].zero_()
    ring.synchronize()
    m, _, _ = ring.acquire(1, hosts[1])
    assert float(m.abs().sum()) == 0.0


def test_offloaded_training_is_bit_identical_and_state_lives_on_the_host():
    e0, cfg = _engine(False)
    e1, _ = _engine(True)
    assert all(u.host_state is not None and u.master.device.type == "cpu" for u in e1.units)
    assert all(u.master.data_ptr() == u.host_state.data_ptr() for u in e1.units)       # views, not copies
    l0, l1 = _train(e0, cfg, 4), _train(e1, cfg, 4)
    assert l0 == l1
    e1.sync_state()
    for a, b in zip(e0.units, e1.units):
        assert torch.equal(a.master, b.master) and torch.equal(a.exp_avg, b.exp_avg)
        assert torch.equal(a.exp_avg_sq, b.exp_avg_sq) and torch.equal(a.compute, b.compute)
    assert float(e0.grad_norm()) == float(e1.grad_norm())
    per_step = sum(u.host_state.numel() for u in e1.units) * 4
    assert e1._offload.h2d_bytes == 4 * per_step and e1._offload.d2h_bytes == 4 * per_step
    # the graph entry point falls back to the eager step instead of capturing host-driven copies
    t = torch.randint(0, cfg.vocab_size, (1, 129))
    e1.graphed_step(t[:, :-1].contiguous(), t[:, 1:].contiguous())
    assert e1.step_count == 5


def test_offloaded_engine_resumes_from_a_checkpoint_of_a_resident_engine_and_back(tmp_path):
    e0, cfg = _engine(False)
    _train(e0, cfg, 2)
    ck = DistributedCheckpointer()
    save_checkpoint(AppState(e0), ck, str(tmp_path / "a"), 2)
    e1, _ = _engine(True, seed=5)
    assert load_checkpoint(AppState(e1), ck, str(tmp_path / "a")) == 2
    _train(e0, cfg, 2, seed=9)
    _train(e1, cfg, 2, seed=9)
    save_checkpoint(AppState(e1), ck, str(tmp_path / "b"), 4)      # saved from host-resident state
    e2, _ = _engine(False, seed=7)
    assert load_checkpoint(AppState(e2), ck, str(tmp_path / "b")) == 4
    for a, b, c in zip(e0.units, e1.units, e2.units):
        assert torch.equal(a.master, b.master) and torch.equal(a.master, c.master)
        assert torch.equal(a.exp_avg_sq, b.exp_avg_sq) and torch.equal(a.exp_avg_sq, c.exp_avg_sq)
        assert torch.equal(a.compute, c.compute)


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _fsdp_worker(rank, world, port, offload, out_q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from ksa_b200.parallel.fsdp import FsdpEngine
        cfg = _cfg()
        model = get_model_class(cfg.model_class)(cfg)
        model.init_weights(seed=0)
        eng = FsdpEngine(model, lr=1e-2, weight_decay=0.1, clip_value=1.0, world_size=world, rank=rank,
                         cpu_offload=offload)
        g = torch.Generator().manual_seed(11)
        data = torch.randint(0, cfg.vocab_size, (3, world, 1, 129), generator=g)
        losses = [float(eng.train_step(data[s, rank][:, :-1].contiguous(), data[s, rank][:, 1:].contiguous()))
                  for s in range(3)]
        eng.sync_state()
        out_q.put((rank, offload, losses, torch.cat([u.compute.clone() for u in eng.units]),
                   torch.cat([u.master.clone() for u in eng.units]), float(eng.grad_norm())))
    finally:
        dist.destroy_process_group()


def test_fsdp_shards_offloaded_on_two_gloo_ranks_match_resident_shards():
    world = 2
    ctx = mp.get_context("spawn")
    res = {}
    for offload in (False, True):
        q = ctx.Queue()
        port = _free_port()
        procs = [ctx.Process(target=_fsdp_worker, args=(r, world, port, offload, q)) for r in range(world)]
        for p in procs:
            p.start()
        got = [q.get(timeout=180) for _ in range(world)]
        for p in procs:
            p.join(timeout=60)
            assert p.exitcode == 0
        res[offload] = sorted(got, key=lambda r: r[0])
    for r in range(world):
        _, _, l0, c0, m0, g0 = res[False][r]
        _, _, l1, c1, m1, g1 = res[True][r]
        assert l0 == l1 and g0 == g1
        assert torch.equal(c0, c1) and torch.equal(m0, m1)
