"""The host-side stream / event model, and the offload staging ring checked with it: the real stream code of
``OptimizerStateOffload`` runs on CPU tensors with recording streams, and no two conflicting accesses may be left
unordered, for any number of units, slots and steps."""
import pytest
import torch

from ksa_b200.training.offload import OptimizerStateOffload, host_state
from ksa_b200.utils.stream_model import Trace, simulated_cuda


def test_the_model_orders_only_what_events_order(monkeypatch):
    with simulated_cuda(monkeypatch) as tr:
        a, b = torch.zeros(8), torch.zeros(8)
        side = torch.cuda.Stream()
        tr.access("produce a", writes=[a])                       # main
        with torch.cuda.stream(side):
            b.copy_(a)                                           # side stream reads a: nothing orders it after main
        assert len(tr.hazards()) == 1 and "write/read" in tr.hazards()[0]
    with simulated_cuda(monkeypatch) as tr:
        a, b = torch.zeros(8), torch.zeros(8)
        side = torch.cuda.Stream()
        tr.access("produce a", writes=[a])
        ev = torch.cuda.Event()
        ev.record(torch.cuda.current_stream())
        side.wait_event(ev)
        with torch.cuda.stream(side):
            b.copy_(a)
        assert tr.hazards() == []
        tr.access("consume b", reads=[b])                        # main again, without waiting for the side stream
        assert len(tr.hazards()) == 1
        torch.cuda.current_stream().wait_stream(side)
        tr.access("consume b again", reads=[b])
        assert len(tr.hazards()) == 1                            # the second read is ordered
        tr.host_access("host looks at b", reads=[b])             # the host never synchronised
        assert len(tr.hazards()) == 2
        side.synchronize()
        tr.host_access("host looks again", reads=[b])
        assert len(tr.hazards()) == 2
        tr.access("disjoint halves", writes=[a[:4]], stream="side1")
        tr.access("disjoint halves", writes=[a[4:]], stream="main")
        assert len(tr.hazards()) == 2                            # no overlap, no hazard


def _ring(tr, n_units, slots, sizes):
    hosts = [host_state(n, torch.device("cpu")) for n in sizes]
    ring = OptimizerStateOffload(torch.device("cpu"), max(sizes), slots=slots)
    ring.cuda = True                                             # take the stream code path, on recording streams
    ring.h2d, ring.d2h = torch.cuda.Stream(), torch.cuda.Stream()
    return ring, hosts


def _steps(tr, ring, hosts, steps, prefetch=True, stream=None):
    for step in range(steps):
        for idx in reversed(range(len(hosts))):
            with torch.cuda.stream(stream) if stream is not None else _null():
                m, a, b = ring.acquire(idx, hosts[idx])
                if prefetch and idx > 0:
                    ring.prefetch(idx - 1, hosts[idx - 1])
                tr.access(f"step {step}: AdamW of unit {idx}", reads=[m, a, b], writes=[m, a, b])
                ring.release(idx, hosts[idx])


class _null:
    def __enter__(self):
        return self

    def __exit__(self, *a):
        return False


@pytest.mark.parametrize("n_units,slots", [(1, 1), (1, 2), (2, 2), (3, 2), (5, 2), (6, 3), (4, 1)])
@pytest.mark.parametrize("prefetch", [True, False])
def test_staging_ring_leaves_no_conflicting_accesses_unordered(monkeypatch, n_units, slots, prefetch):
    sizes = [5 + 3 * i for i in range(n_units)]
    with simulated_cuda(monkeypatch) as tr:
        ring, hosts = _ring(tr, n_units, slots, sizes)
        comm = torch.cuda.Stream()                               # the sharded engine updates on its side stream
        _steps(tr, ring, hosts, 2, prefetch)
        _steps(tr, ring, hosts, 2, prefetch, stream=comm)
        ring.synchronize()
        tr.host_access("checkpoint reads the state", reads=hosts)
        tr.host_access("a load overwrites the state", writes=hosts)
        _steps(tr, ring, hosts, 1, prefetch)
        assert tr.hazards() == [], tr.hazards()[:3]
        copies = [o for o in tr.ops if o.what == "copy"]
        assert len(copies) == 2 * 5 * n_units                    # every unit in and out once per step


def test_the_model_catches_a_ring_that_forgets_an_ordering(monkeypatch):
    # 1. slots reused without waiting for the write-back of their last tenant
    with simulated_cuda(monkeypatch) as tr:
        ring, hosts = _ring(tr, 4, 2, [8, 8, 8, 8])
        real_release = ring.release

        def forgetful_release(idx, host):
            real_release(idx, host)
            ring._written = [None] * ring.slots
        ring.release = forgetful_release
        _steps(tr, ring, hosts, 1)
        assert any("read/write" in h or "write/read" in h for h in tr.hazards())
    # 2. the host reads the state without synchronising with the write-back stream
    with simulated_cuda(monkeypatch) as tr:
        ring, hosts = _ring(tr, 2, 2, [8, 8])
        _steps(tr, ring, hosts, 1)
        tr.host_access("checkpoint without synchronize()", reads=hosts)
        assert any("host" in h for h in tr.hazards())
    # 3. the update starts without waiting for its load
    with simulated_cuda(monkeypatch) as tr:
        ring, hosts = _ring(tr, 2, 2, [8, 8])
        ring.prefetch(1, hosts[1])
        v = ring._view(1, hosts[1])
        tr.access("AdamW without acquire()", reads=[v], writes=[v])
        assert any("write/read" in h or "write/write" in h for h in tr.hazards())


@pytest.mark.parametrize("offload", [False, True])
@pytest.mark.parametrize("accum", [1, 2])
def test_single_gpu_engine_with_the_optimizer_under_the_backward_pass(monkeypatch, offload, accum):
    """``TrainEngine(overlap_optimizer=True)`` (and the staging ring with it, when the state is offloaded) on
    recording streams: every unit's AdamW runs on the side stream between the backward pass of its layer and the next
    forward pass, and every conflicting pair of accesses is ordered by an event."""
    from ksa_b200.config import get_preset
    from ksa_b200.models import get_model_class
    from ksa_b200.training.engine import TrainEngine
    cfg = get_preset("qwen3-ksa-tiny").merge({"num_layers": 3, "summary_layer_freq": [1, 0, 1], "embed_dim": 64,
                                               "intermediate_dim": 128, "vocab_size": 256, "head_dim": 16})
    model = get_model_class(cfg.model_class)(cfg)
    model.init_weights(seed=0)
    with simulated_cuda(monkeypatch) as tr:
        eng = TrainEngine(model, lr=1e-2, weight_decay=0.1, clip_value=1.0, grad_accum_steps=accum,
                          overlap_optimizer=True, cpu_offload=offload)
        eng.opt_stream = torch.cuda.Stream()                     # take the stream code path, on recording streams
        if offload:
            eng._offload.cuda = True
            eng._offload.h2d, eng._offload.d2h = torch.cuda.Stream(), torch.cuda.Stream()
        names = [u.name for u in eng.units]
        for i, layer in enumerate(model.get_layers_to_shard()):
            u = eng.units[names.index(f"layer{i}")]
            layer.register_forward_pre_hook(lambda m, a, u=u: tr.access(f"forward pass of {u.name}", reads=[u.compute]))
            layer.register_full_backward_pre_hook(
                lambda m, g, u=u: tr.access(f"backward pass of {u.name}", reads=[u.compute], writes=[u.grad]))
        plain = eng._reduce_and_update

        def logged(u):
            with eng._optimizer_state(u) as state:               # the views the kernel would get (a staging slot)
                tr.access(f"AdamW of {u.name}", reads=[u.grad, *state], writes=[*state, u.compute])
                if eng._offload is None:
                    return plain(u)
                from ksa_b200 import ops
                ops.adamw_step(*state[:1], u.grad, *state[1:], None, eng.hyper, eng.beta1, eng.beta2, eng.eps,
                               eng.weight_decay, eng.clip_value, eng.grad_sq)
                u.compute.copy_(state[0])
        eng._reduce_and_update = logged
        g = torch.Generator().manual_seed(3)
        for _ in range(3 * accum):
            t = torch.randint(0, cfg.vocab_size, (2, 129), generator=g)
            eng.train_step(t[:, :-1].contiguous(), t[:, 1:].contiguous())
        eng.sync_state()
        if offload:      # the state is host memory: the host reads it directly, after sync_state()
            tr.host_access("checkpoint", reads=[u.master for u in eng.units])
        else:            # device memory leaves through a copy on the main stream
            tr.access("checkpoint copy", reads=[u.master for u in eng.units])
        assert tr.hazards() == [], tr.hazards()[:4]
        side = [o for o in tr.ops if o.what.startswith("AdamW") and o.stream != "main"]
        assert len(side) == 3 * 4 and eng.step_count == 3        # head + three layers per step on the side stream
    # the same schedule with the join at the end of the optimizer step taken away must be reported
    model2 = get_model_class(cfg.model_class)(cfg)
    model2.init_weights(seed=0)
    with simulated_cuda(monkeypatch) as tr:
        from ksa_b200.utils import stream_model
        monkeypatch.setattr(stream_model._Stream, "wait_stream", lambda self, other: None)
        eng = TrainEngine(model2, lr=1e-2, overlap_optimizer=True)
        eng.opt_stream = torch.cuda.Stream()
        names = [u.name for u in eng.units]
        for i, layer in enumerate(model2.get_layers_to_shard()):
            u = eng.units[names.index(f"layer{i}")]
            layer.register_forward_pre_hook(lambda m, a, u=u: tr.access(f"forward pass of {u.name}", reads=[u.compute]))
        plain2 = eng._reduce_and_update
        eng._reduce_and_update = lambda u: (tr.access(f"AdamW of {u.name}", reads=[u.grad], writes=[u.compute]), plain2(u))
        for _ in range(2):
            t = torch.randint(0, cfg.vocab_size, (2, 129), generator=g)
            eng.train_step(t[:, :-1].contiguous(), t[:, 1:].contiguous())
        assert any("AdamW of layer" in h and "forward pass" in h for h in tr.hazards())


def test_staging_ring_under_arbitrary_orders_of_units_and_prefetches(monkeypatch):
    """Any order of updates, any prefetch hints (also useless or conflicting ones), one to three slots: no hazard, and
    every unit's values survive the round trips (each update adds 1 to the master row)."""
    from hypothesis import given, settings, strategies as st

    @settings(max_examples=60, deadline=None)
    @given(slots=st.integers(1, 3), n_units=st.integers(1, 6),
           order=st.lists(st.tuples(st.integers(0, 5), st.one_of(st.none(), st.integers(0, 5))), min_size=1, max_size=25))
    def run(slots, n_units, order):
        with monkeypatch.context() as mp:
            with simulated_cuda(mp) as tr:
                ring, hosts = _ring(tr, n_units, slots, [4 + i for i in range(n_units)])
                counts = [0] * n_units
                for idx, hint in order:
                    idx %= n_units
                    m, a, b = ring.acquire(idx, hosts[idx])
                    if hint is not None and hint % n_units != idx:
                        ring.prefetch(hint % n_units, hosts[hint % n_units])
                    tr.access(f"AdamW of unit {idx}", reads=[m, a, b], writes=[m, a, b])
                    m += 1.0
                    counts[idx] += 1
                    ring.release(idx, hosts[idx])
                ring.synchronize()
                tr.host_access("checkpoint", reads=hosts)
                assert tr.hazards() == [], tr.hazards()[:3]
                for i, h in enumerate(hosts):
                    assert float(h[0].min()) == float(h[0].max()) == float(counts[i]), (i, counts, h[0])
                    assert float(h[1:].abs().sum()) == 0.0
    run()
