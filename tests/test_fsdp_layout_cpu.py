"""The fused FSDP back end (``ksa_b200/parallel/fsdp.py`` with ``comm="fused"``: symmetric parameter and gradient
buffers, per-unit flags, pull all-gather, reduce-scatter + AdamW on the shard owner) on 2, 4 and 8 ranks without a GPU.

Every rank is a thread with its own engine; symmetric buffers are CPU tensors reachable through their addresses and
the communication kernels are Python stand-ins that honour the same pointers, shard ranges, hyper-parameter vector and
flag values.  On CPU the weight gradients reach the fp32 buffers only after backward (autograd ``.grad``), so the
hooks that start a unit's reduction in the middle of backward are switched off and every unit is reduced at the
optimizer step: what is checked is the sharding, the flag protocol and the gather schedule of each overlap mode, not
the overlap itself.  The result is compared with single-process training on the same micro-batches.
"""
import contextlib
import copy

import pytest
import torch
import torch.distributed as dist

from ksa_b200.models import get_model_class
from ksa_b200.ops import _lib
from ksa_b200.parallel import symm
from ksa_b200.parallel.fsdp import FsdpEngine
from ksa_b200.training.engine import TrainEngine

from test_cp_layout_cpu import ZeroedSymm, _raw, make_cp_kernels
from test_fsdp_cpu import _tiny
from test_tp_layout_cpu import _FakeEvent, _FakeStream, _ptrs, _run_ranks


def make_fsdp_kernels(mem, log):
    base = make_cp_kernels(mem, log)          # ksa_signal_set / ksa_signal_wait and the flag helpers' semantics

    def flag_value(ptr):
        return int(_raw(mem, ptr, 4).view(torch.int32)[0])

    def wait(ptr, target):
        import time
        t0 = time.monotonic()
        while flag_value(ptr) < target:
            if time.monotonic() - t0 > 60:
                raise AssertionError(f"a wait for flag value {target} ran out (flag holds {flag_value(ptr)})")
            time.sleep(0.0005)

    def target_of(epoch, add):
        return (int(epoch[0]) if epoch is not None else 0) + add

    def call(name, *a):
        if name == "ksa_peer_gather":
            log.append(name)
            ptrs, world, rank, shard_elems, elem_bytes, ready, epoch, add, _ctas = a
            ptrs, n = _ptrs(ptrs, world), shard_elems * elem_bytes
            for step in range(1, world):
                r = (rank + step) % world
                if ready is not None:
                    wait(ready + 4 * r, target_of(epoch, add))
                _raw(mem, ptrs[rank] + r * n, n).copy_(_raw(mem, ptrs[r] + r * n, n))
        elif name == "ksa_peer_reduce_adamw":
            log.append(name)
            (grads, world, rank, shard_lo, n, master, m, v, out, hyper, b1, b2, eps, wd, clip, sumsq, ready, epoch, add,
             _ctas) = a
            if ready is not None:
                for r in range(world):
                    wait(ready + 4 * r, target_of(epoch, add))
            g = torch.zeros(n)
            for p in _ptrs(grads, world):
                g += _raw(mem, p + 4 * shard_lo, 4 * n).view(torch.float32)
            lr, bc1, bc2, gscale = (float(x) for x in hyper)
            g = g * gscale
            if sumsq is not None:
                sumsq += (g * g).sum()
            if clip > 0:
                g = g.clamp(-clip, clip)
            m.mul_(b1).add_(g, alpha=1 - b1)
            v.mul_(b2).addcmul_(g, g, value=1 - b2)
            master.mul_(1 - lr * wd).sub_(lr * (m / bc1) / ((v / bc2).sqrt() + eps))
            if isinstance(out, int):      # resharded storage: an address that shard_lo elements (bf16) are added to
                _raw(mem, out + 2 * shard_lo, 2 * n).view(torch.bfloat16).copy_(master)
            elif out is not None:
                out[shard_lo:shard_lo + n].copy_(master)
        else:
            base(name, *a)
    return call


@pytest.fixture
def fake_fsdp_gpu(monkeypatch):
    monkeypatch.setattr(symm, "SymmetricBuffer", ZeroedSymm)
    monkeypatch.setattr(dist, "get_rank", lambda g=None: g.rank)
    monkeypatch.setattr(dist, "get_world_size", lambda g=None: g.size)
    monkeypatch.setattr(torch.cuda, "synchronize", lambda device=None: None)
    monkeypatch.setattr(torch.cuda, "Stream", lambda device=None: _FakeStream())
    monkeypatch.setattr(torch.cuda, "current_stream", lambda device=None: _FakeStream())
    monkeypatch.setattr(torch.cuda, "stream", lambda s: contextlib.nullcontext())
    monkeypatch.setattr(torch.cuda, "Event", lambda **kw: _FakeEvent())
    monkeypatch.setattr(torch.cuda, "is_current_stream_capturing", lambda: False)
    # CPU autograd fills .grad after the boundary hooks have fired: reduce every unit at the optimizer step instead
    monkeypatch.setattr(FsdpEngine, "_backward_reached", lambda self, tag: None)
    yield


@pytest.mark.parametrize("world,overlap,reshard", [(2, "stream", False), (2, "gemm2", False), (4, "stream", False),
                                                   (4, "gemm2", False), (8, "stream", False), (2, "stream", True),
                                                   (4, "stream", True)])
def test_fused_fsdp_matches_single_process_training(fake_fsdp_gpu, monkeypatch, world, overlap, reshard):
    """``reshard``: ZeRO-3 storage (bf16 shards + a pool of slots that units share); six layers so that every layer slot
    gets a second and a third tenant in forward and has to be refilled in backward."""
    steps = 3
    cfg = _tiny() if not reshard else _tiny().merge({"num_layers": 6, "summary_layer_freq": [1, 1, 0, 1, 1, 0]})
    torch.manual_seed(0)
    base = get_model_class(cfg.model_class)(cfg)
    base.init_weights(seed=0)
    base = base.to(torch.bfloat16)
    g = torch.Generator().manual_seed(7)
    data = torch.randint(0, cfg.vocab_size, (steps, world, 1, 257), generator=g)
    log, results = [], {}

    def body(rank, group):
        if rank == 0:
            monkeypatch.setattr(_lib, "call", make_fsdp_kernels(group.shared["mem"], log))
        group.shared["barrier"].wait()
        model = copy.deepcopy(base)
        eng = FsdpEngine(model, lr=1e-2, weight_decay=0.1, clip_value=1.0, world_size=world, rank=rank, group=group,
                         comm="fused", overlap=overlap, param_dtype=torch.bfloat16, device="cpu",
                         pair_gather_min_flops=0.0, reshard_after_forward=reshard)
        if reshard:
            # bf16 weights held: 1/world of the model + three layer slots + one slot for the embedding / head
            lay = max(u.size for u in eng.units if u.name.startswith("layer"))
            big = max(u.size for u in eng.units if not u.name.startswith("layer"))
            want = sum(u.size for u in eng.units) // world * 2 + (big + 3 * lay) * 2
            assert want <= eng.compute_weight_bytes() <= want + 512, (eng.compute_weight_bytes(), want)
        losses = []
        for s in range(steps):
            t = data[s, rank]
            losses.append(float(eng.train_step(t[:, :-1].contiguous(), t[:, 1:].contiguous())))
        group.shared["barrier"].wait()
        eng._write_hyper()                   # pull the last update of every unit, as the next forward would
        eng._overlap_active = False
        final = {}
        for ui in range(len(eng.units)):     # unit by unit: with resharded storage several units share a slot
            eng._gather_now(ui)
            final.update({s.name: s.param.detach().float().clone() for s in eng.units[ui].slots})
        group.shared["barrier"].wait()
        results[rank] = (losses, final, float(eng.grad_sq))
        eng.close()

    _run_ranks(world, body)
    ref_model = copy.deepcopy(base)
    ref = TrainEngine(ref_model, lr=1e-2, weight_decay=0.1, clip_value=1.0, grad_accum_steps=world,
                      param_dtype=torch.bfloat16)
    ref_losses = []
    for s in range(steps):
        for r in range(world):
            t = data[s, r]
            ref_losses.append(float(ref.train_step(t[:, :-1].contiguous(), t[:, 1:].contiguous())))
    for r in range(world):
        for s in range(steps):
            assert abs(results[r][0][s] - ref_losses[s * world + r]) < 3e-2, (r, s, results[r][0], ref_losses)
    want = {n: p.detach().float() for n, p in ref_model.named_parameters()}
    for r in range(world):
        for n, w in want.items():
            got = results[r][1][n]
            # The single process adds its micro-batch gradients up in bf16 (.grad), the ranks' gradients are summed in
            # fp32: where the sum is close to zero the first Adam steps (size lr, sign of the gradient) can differ.
            # A shard that was not reduced, updated or gathered would be off in a quarter or more of the elements.
            off = int(((got - w).abs() > 1.2e-2).sum())       # more than one step of size lr, or one bf16 ulp at 1.0
            assert off <= max(2, got.numel() // 100), (r, n, off, got.numel())
            assert (got - w).norm() <= 6e-2 * w.norm().clamp_min(1e-3), (r, n, float((got - w).norm()), float(w.norm()))
            assert torch.equal(got, results[0][1][n]), f"ranks disagree about {n}"
    total_sq = sum(results[r][2] for r in range(world))        # every rank holds the sum over its shards
    assert abs(total_sq ** 0.5 - float(ref.grad_norm())) < 5e-2 * float(ref.grad_norm())
    assert "ksa_peer_gather" in log and "ksa_peer_reduce_adamw" in log and "ksa_signal_set" in log


def test_context_parallel_and_fsdp_on_the_same_ranks(fake_fsdp_gpu, monkeypatch):
    """The long-context configuration: 4 ranks split every sequence (fused context-parallel exchange) and shard the
    weights (fused FSDP) at the same time; two optimizer steps equal single-process training on the whole sequences."""
    from test_cp_cpu import _cfg
    from test_cp_layout_cpu import apply_cp_patches
    from ksa_b200.parallel.cp import CpContext, shard_inputs
    apply_cp_patches(monkeypatch)
    world, L, chunk, window, n_sum, B, steps = 4, 128, 16, 3, 1, 2, 2
    cfg = _cfg(chunk, window, n_sum)
    torch.manual_seed(0)
    base = get_model_class(cfg.model_class)(cfg)
    base.init_weights(seed=0)
    base = base.to(torch.bfloat16)
    g = torch.Generator().manual_seed(3)
    data = torch.randint(0, 200, (steps, B, L + 1), generator=g)
    log, results = [], {}

    def body(rank, group):
        if rank == 0:
            monkeypatch.setattr(_lib, "call", make_fsdp_kernels(group.shared["mem"], log))
        group.shared["barrier"].wait()
        model = copy.deepcopy(base)
        model.cp = CpContext(group, L, chunk, n_sum, cfg.num_kv_heads, cfg.head_dim, batch=B, device="cuda",
                             dtype=torch.bfloat16, n_heads=cfg.num_heads, full_layers=True, max_window=window,
                             full_layer_mode="halo")
        eng = FsdpEngine(model, lr=1e-2, weight_decay=0.1, clip_value=1.0, world_size=world, rank=rank, group=group,
                         comm="fused", overlap="stream", param_dtype=torch.bfloat16, device="cpu")
        losses = []
        for s in range(steps):
            tokens, labels = shard_inputs(data[s, :, :-1], data[s, :, 1:], rank, world)
            losses.append(float(eng.train_step(tokens, labels)))
        group.shared["barrier"].wait()
        eng._write_hyper()
        eng._overlap_active = False
        for ui in range(len(eng.units)):
            eng._gather_now(ui)
        group.shared["barrier"].wait()
        results[rank] = (losses, {n: p.detach().float().clone() for n, p in model.named_parameters()})
        eng.close()
        model.cp.close()

    _run_ranks(world, body)
    ref_model = copy.deepcopy(base)
    ref = TrainEngine(ref_model, lr=1e-2, weight_decay=0.1, clip_value=1.0, param_dtype=torch.bfloat16)
    ref_losses = [float(ref.train_step(data[s, :, :-1].contiguous(), data[s, :, 1:].contiguous())) for s in range(steps)]
    for s in range(steps):
        assert abs(sum(results[r][0][s] for r in range(world)) / world - ref_losses[s]) < 3e-2
    want = {n: p.detach().float() for n, p in ref_model.named_parameters()}
    for r in range(world):
        for n, w in want.items():
            got = results[r][1][n]
            off = int(((got - w).abs() > 1.2e-2).sum())
            assert off <= max(2, got.numel() // 50), (r, n, off, got.numel())
            assert torch.equal(got, results[0][1][n]), f"ranks disagree about {n}"
    assert "ksa_peer_copy" in log and "ksa_peer_reduce_adamw" in log and "ksa_peer_add_bf16" in log


@pytest.mark.parametrize("world,overlap,reshard,broken", [
    (2, "stream", False, None), (2, "stream", True, None), (3, "stream", True, None), (2, "gemm2", False, None),
    (2, "stream", True, "wait_event"), (2, "stream", True, "wait_stream")])
def test_fused_fsdp_stream_schedule_orders_every_conflicting_access(fake_fsdp_gpu, monkeypatch, world, overlap, reshard,
                                                                    broken):
    """The host-side stream model over the fused engine's real schedule: gathers one unit ahead on the side stream,
    units reduced and updated on the side stream while the backward pass runs, ZeRO-3 slots with several tenants.
    Every rank records its copies, its kernels' accesses to its own buffers and the reads / writes of the forward and
    backward pass of each unit; no pair of conflicting accesses on different streams may be left without an event
    between them.  (Accesses to other ranks' memory are ordered by device-side flags, not by streams: not modelled.)
    Here the hooks that update a unit in the middle of the backward pass stay on: the numbers are not checked (on CPU
    the gradients arrive later), only the order of the launches.  ``broken`` takes one kind of ordering away from the
    streams: the check must then report conflicts (it is not satisfied by anything)."""
    from ksa_b200.utils import stream_model
    from ksa_b200.utils.stream_model import SimulatedCuda
    monkeypatch.undo()                        # the fixture's blanket patches; re-applied below without the two we replace
    monkeypatch.setattr(symm, "SymmetricBuffer", ZeroedSymm)
    monkeypatch.setattr(dist, "get_rank", lambda g=None: g.rank)
    monkeypatch.setattr(dist, "get_world_size", lambda g=None: g.size)
    monkeypatch.setattr(torch.cuda, "synchronize", lambda device=None: None)
    monkeypatch.setattr(torch.cuda, "is_current_stream_capturing", lambda: False)
    sim = SimulatedCuda(per_thread=True)
    sim.install(monkeypatch)
    if broken:
        monkeypatch.setattr(stream_model._Stream, broken, lambda self, other: None)
    cfg = _tiny().merge({"num_layers": 6, "summary_layer_freq": [1, 1, 0, 1, 1, 0]})
    torch.manual_seed(0)
    base = get_model_class(cfg.model_class)(cfg)
    base.init_weights(seed=0)
    base = base.to(torch.bfloat16)
    data = torch.randint(0, cfg.vocab_size, (3, world, 1, 257), generator=torch.Generator().manual_seed(7))
    log, results = [], {}

    def logging_kernels(mem):
        inner = make_fsdp_kernels(mem, log)

        def call(name, *a):
            tr = sim.trace
            if name == "ksa_peer_gather":
                ptrs, w, rank, shard_elems, elem_bytes = a[0], a[1], a[2], a[3], a[4]
                n = shard_elems * elem_bytes
                mine = _ptrs(ptrs, w)[rank]
                tr.access("gather kernel", writes=[_raw(mem, mine + r * n, n) for r in range(w) if r != rank])
            elif name == "ksa_peer_reduce_adamw":
                grads, w, rank, shard_lo, n, master, m, v, out = a[:9]
                writes = [master, m, v]
                if isinstance(out, int):
                    writes.append(_raw(mem, out + 2 * shard_lo, 2 * n))
                elif out is not None:
                    writes.append(out[shard_lo:shard_lo + n])
                tr.access("reduce + AdamW kernel", reads=[_raw(mem, _ptrs(grads, w)[rank] + 4 * shard_lo, 4 * n)],
                          writes=writes)
            return inner(name, *a)
        return call

    def body(rank, group):
        tr = sim.enter_thread()
        if rank == 0:
            monkeypatch.setattr(_lib, "call", logging_kernels(group.shared["mem"]))
        group.shared["barrier"].wait()
        with sim.log_copies():
            model = copy.deepcopy(base)
            eng = FsdpEngine(model, lr=1e-2, weight_decay=0.1, clip_value=1.0, world_size=world, rank=rank,
                             group=group, comm="fused", overlap=overlap, param_dtype=torch.bfloat16, device="cpu",
                             pair_gather_min_flops=0.0, reshard_after_forward=reshard)
            for i, layer in enumerate(model.get_layers_to_shard()):
                u = eng.units[eng._layer_unit[i]]
                layer.register_forward_pre_hook(
                    lambda m, a, u=u: tr.access(f"forward pass of {u.name}", reads=[u.compute]))
                layer.register_full_backward_pre_hook(
                    lambda m, g, u=u: tr.access(f"backward pass of {u.name}", reads=[u.compute], writes=[u.grad]))
            for s in range(3):
                t = data[s, rank]
                eng.train_step(t[:, :-1].contiguous(), t[:, 1:].contiguous())
            group.shared["barrier"].wait()
            results[rank] = (tr.hazards(), len(tr.ops), sorted({o.stream for o in tr.ops}))
            eng.close()

    _run_ranks(world, body)
    for rank in range(world):
        hazards, n_ops, streams = results[rank]
        if broken:
            assert hazards and any("[side1]" in h and "[main]" in h for h in hazards), (rank, broken)
        else:
            assert hazards == [], (rank, hazards[:4])
        assert n_ops > 100 and len(streams) >= 2, (n_ops, streams)      # the side stream did carry work
    assert "ksa_peer_gather" in log and "ksa_peer_reduce_adamw" in log
