"""A host-side model of CUDA streams and events for checking stream choreography without a GPU.

Code that orders copies and kernels with ``torch.cuda.Stream`` / ``torch.cuda.Event`` runs unchanged on CPU tensors
inside :func:`simulated_cuda`: streams and events are replaced by recording stand-ins, every ``Tensor.copy_`` is logged
with the stream that was current and the memory it read and wrote, and callers log the accesses of their kernels with
:meth:`Trace.access`.  :meth:`Trace.hazards` then asks the one question that matters: is every pair of accesses to
overlapping memory (at least one of them a write) that were issued on different streams ordered by an event?  Streams
run asynchronously, so host issue order alone orders nothing; only ``record`` -> ``wait_event``, ``wait_stream`` and
``synchronize`` do.  Vector clocks (one component per stream) decide it.

compute-sanitizer's racecheck cannot be run where this package is developed; this model covers the host-side half of
the same question (which launches and copies may overlap), the bounded device-side waits cover the other half.
"""
from __future__ import annotations

import contextlib
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple

import torch
from torch.overrides import TorchFunctionMode

__all__ = ["Trace", "SimulatedCuda", "simulated_cuda", "span"]


def span(t: torch.Tensor) -> Tuple[int, int]:
    """Address range ``[lo, hi)`` that a (possibly strided) tensor can touch."""
    if t.numel() == 0:
        return (t.data_ptr(), t.data_ptr())
    extent = 1 + sum((s - 1) * abs(st) for s, st in zip(t.shape, t.stride()))
    return (t.data_ptr(), t.data_ptr() + extent * t.element_size())


@dataclass
class _Op:
    index: int
    stream: str
    what: str
    reads: List[Tuple[int, int]]
    writes: List[Tuple[int, int]]
    clock: Dict[str, int]


@dataclass
class Trace:
    ops: List[_Op] = field(default_factory=list)
    clocks: Dict[str, Dict[str, int]] = field(default_factory=dict)       # stream -> what it has seen of every stream
    current: List[str] = field(default_factory=lambda: ["main"])

    # ------------------------------------------------------------------ clocks
    def _clock(self, stream: str) -> Dict[str, int]:
        return self.clocks.setdefault(stream, {})

    @staticmethod
    def _join(into: Dict[str, int], other: Dict[str, int]) -> None:
        for k, v in other.items():
            if v > into.get(k, 0):
                into[k] = v

    def access(self, what: str, reads=(), writes=(), stream: Optional[str] = None) -> None:
        """Log work issued on ``stream`` (default: the current one) that reads / writes the given tensors."""
        s = stream or self.current[-1]
        c = self._clock(s)
        if s != "host":      # work is launched after everything the host thread did itself before the launch
            c["host"] = self._clock("host").get("host", 0)
        c[s] = c.get(s, 0) + 1
        self.ops.append(_Op(len(self.ops), s, what, [span(t) for t in reads], [span(t) for t in writes], dict(c)))

    def host_access(self, what: str, reads=(), writes=()) -> None:
        """The host thread touches memory itself (no stream): ordered only by ``synchronize`` calls before it."""
        self.access(what, reads, writes, stream="host")

    # ------------------------------------------------------------------ verdict
    def hazards(self) -> List[str]:
        """Unordered conflicting pairs, as readable lines (empty: the choreography is race-free)."""
        out = []
        for j, b in enumerate(self.ops):
            for a in self.ops[:j]:
                if a.stream == b.stream:
                    continue
                if a.clock[a.stream] <= b.clock.get(a.stream, 0):
                    continue                                    # b has seen a
                kinds = []
                if _overlap(a.writes, b.writes):
                    kinds.append("write/write")
                if _overlap(a.writes, b.reads):
                    kinds.append("write/read")
                if _overlap(a.reads, b.writes):
                    kinds.append("read/write")
                if kinds:
                    out.append(f"{'+'.join(kinds)}: #{a.index} {a.what} [{a.stream}] is not ordered before "
                               f"#{b.index} {b.what} [{b.stream}]")
        return out


def _overlap(xs, ys) -> bool:
    return any(a[0] < b[1] and b[0] < a[1] for a in xs for b in ys)


class _Stream:
    def __init__(self, trace: Trace, name: str):
        self.trace, self.name = trace, name

    def wait_event(self, ev: "_Event") -> None:
        if ev.clock is not None:
            Trace._join(self.trace._clock(self.name), ev.clock)

    def wait_stream(self, other: "_Stream") -> None:
        Trace._join(self.trace._clock(self.name), self.trace._clock(other.name))

    def record_event(self, ev: Optional["_Event"] = None) -> "_Event":
        ev = ev or _Event(self.trace)
        ev.record(self)
        return ev

    def synchronize(self) -> None:
        Trace._join(self.trace._clock("host"), self.trace._clock(self.name))


class _Event:
    def __init__(self, trace: Trace, *a, **kw):
        self.trace, self.clock = trace, None

    def record(self, stream: Optional[_Stream] = None) -> None:
        name = stream.name if stream is not None else self.trace.current[-1]
        self.clock = dict(self.trace._clock(name))

    def synchronize(self) -> None:
        if self.clock is not None:
            Trace._join(self.trace._clock("host"), self.clock)

    def wait(self, stream: Optional[_Stream] = None) -> None:
        name = stream.name if stream is not None else self.trace.current[-1]
        if self.clock is not None:
            Trace._join(self.trace._clock(name), self.clock)


class _LogCopies(TorchFunctionMode):
    def __init__(self, trace: Trace):
        super().__init__()
        self.trace = trace

    def __torch_function__(self, func, types, args=(), kwargs=None):
        kwargs = kwargs or {}
        if func is torch.Tensor.copy_ and len(args) >= 2 and isinstance(args[1], torch.Tensor):
            self.trace.access("copy", reads=[args[1]], writes=[args[0]])
        return func(*args, **kwargs)


class SimulatedCuda:
    """The stand-ins behind :func:`simulated_cuda`.  With ``per_thread=True`` every thread (a rank of a CPU emulation)
    gets its own :class:`Trace` and its own streams: call :meth:`enter_thread` in each of them."""

    def __init__(self, per_thread: bool = False):
        import threading
        self.per_thread = per_thread
        self._local = threading.local() if per_thread else type("_Shared", (), {})()
        self._lock = threading.Lock()
        self.traces: List[Trace] = []

    def enter_thread(self, trace: Optional[Trace] = None) -> Trace:
        loc = self._local
        loc.trace = trace or Trace()
        loc.streams = {"main": _Stream(loc.trace, "main")}
        loc.count = 0
        with self._lock:
            self.traces.append(loc.trace)
        return loc.trace

    @property
    def trace(self) -> Trace:
        return self._local.trace

    def new_stream(self, *a, **kw) -> _Stream:
        loc = self._local
        loc.count += 1
        s = _Stream(loc.trace, f"side{loc.count}")
        loc.streams[s.name] = s
        return s

    def new_event(self, *a, **kw) -> _Event:
        return _Event(self._local.trace)

    @contextlib.contextmanager
    def use(self, stream):
        cur = self._local.trace.current
        cur.append(stream.name)
        try:
            yield
        finally:
            cur.pop()

    def current_stream(self, *a, **kw) -> _Stream:
        loc = self._local
        return loc.streams[loc.trace.current[-1]]

    def install(self, monkeypatch) -> None:
        monkeypatch.setattr(torch.cuda, "Stream", self.new_stream)
        monkeypatch.setattr(torch.cuda, "Event", self.new_event)
        monkeypatch.setattr(torch.cuda, "stream", self.use)
        monkeypatch.setattr(torch.cuda, "current_stream", self.current_stream)

    def log_copies(self):
        """Context manager (per thread) that logs every ``Tensor.copy_`` into this thread's trace."""
        return _LogCopies(self._local.trace)


@contextlib.contextmanager
def simulated_cuda(monkeypatch, trace: Optional[Trace] = None):
    """Replace ``torch.cuda.Stream / Event / stream / current_stream`` by recording stand-ins (through pytest's
    ``monkeypatch``) and log every ``Tensor.copy_``; yields the :class:`Trace`."""
    sim = SimulatedCuda()
    trace = sim.enter_thread(trace)
    sim.install(monkeypatch)
    with sim.log_copies():
        yield trace
