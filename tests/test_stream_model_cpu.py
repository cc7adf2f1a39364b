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
