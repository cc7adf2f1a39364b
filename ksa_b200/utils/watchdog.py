"""Failure detection around the training loop (the reference has none beyond a 24-hour process-group timeout,
``recipes/pretrain_kai_summary_unified.py:22``, and restart-from-``latest``).

Three host-side pieces, none of which touches a GPU:

* :class:`StepWatchdog` - a thread that expects ``beat()`` once per step and reports a stall after ``timeout_s``.
* :class:`HeartbeatMonitor` - every rank publishes a heartbeat (and, on failure, an ``abort`` record) in a key-value
  store (``torch.distributed.TCPStore``/``FileStore``/``HashStore``); ``check()`` is called *between* steps, before
  the next kernels or collectives are launched, so that a surviving rank stops cleanly instead of waiting for a peer
  that will never arrive.
* :class:`FaultInjector` - host-side fault injection for tests: raise, exit or stall on a chosen rank and step,
  driven by the ``KSA_FAULT`` environment variable (``"raise@step=3,rank=1"``).

Device-side waits (peer flags, mbarriers) are bounded inside the kernels and report through a status word that
``ksa_b200.ops._lib.check_status`` turns into an exception; :func:`check_device` wraps that for the loop.
"""
from __future__ import annotations

import os
import sys
import threading
import time
import traceback
from dataclasses import dataclass
from typing import Callable, Dict, List, Optional


class RankFailure(RuntimeError):
    """Another rank reported a failure or stopped sending heartbeats."""


class StepStall(RuntimeError):
    """No step finished within the watchdog's limit."""


class StepWatchdog:
    def __init__(self, timeout_s: float, on_timeout: Optional[Callable[[float], None]] = None, poll_s: float = 0.5):
        self.timeout_s = timeout_s
        self.on_timeout = on_timeout or self._default
        self.poll_s = min(poll_s, max(timeout_s / 4, 0.01))
        self._last = time.monotonic()
        self._stop = threading.Event()
        self.fired = False
        self._thread = threading.Thread(target=self._run, name="ksa-step-watchdog", daemon=True)

    def _default(self, idle: float) -> None:
        print(f"[watchdog] no training step finished for {idle:.0f} s; stacks of all threads follow", file=sys.stderr)
        for tid, frame in sys._current_frames().items():
            print(f"--- thread {tid}", file=sys.stderr)
            traceback.print_stack(frame, file=sys.stderr)

    def start(self) -> "StepWatchdog":
        self._last = time.monotonic()
        self._thread.start()
        return self

    def beat(self) -> None:
        self._last = time.monotonic()

    def stop(self) -> None:
        self._stop.set()
        if self._thread.is_alive():
            self._thread.join(timeout=2 * self.poll_s + 1)

    def _run(self) -> None:
        while not self._stop.wait(self.poll_s):
            idle = time.monotonic() - self._last
            if idle > self.timeout_s and not self.fired:
                self.fired = True
                try:
                    self.on_timeout(idle)
                finally:
                    pass

    def __enter__(self):
        return self.start()

    def __exit__(self, *exc):
        self.stop()


class HeartbeatMonitor:
    """Heartbeats and abort records in a ``torch.distributed`` store."""

    def __init__(self, store, rank: int, world_size: int, timeout_s: float = 120.0, prefix: str = "ksa_hb"):
        self.store, self.rank, self.world, self.timeout_s, self.prefix = store, rank, world_size, timeout_s, prefix
        self._seen: Dict[int, float] = {}
        self.beat(step=-1)

    def _key(self, kind: str, rank: int) -> str:
        return f"{self.prefix}/{kind}/{rank}"

    def beat(self, step: int) -> None:
        self.store.set(self._key("beat", self.rank), f"{step}:{time.time():.3f}")

    def report_failure(self, reason: str) -> None:
        self.store.set(self._key("abort", self.rank), reason[:500])

    def _get(self, key: str) -> Optional[str]:
        try:
            if hasattr(self.store, "check") and not self.store.check([key]):
                return None
            return self.store.get(key).decode()
        except Exception:
            return None

    def failed_ranks(self) -> Dict[int, str]:
        out: Dict[int, str] = {}
        now = time.time()
        for r in range(self.world):
            if r == self.rank:
                continue
            reason = self._get(self._key("abort", r))
            if reason is not None:
                out[r] = "reported: " + reason
                continue
            beat = self._get(self._key("beat", r))
            if beat is None:
                first = self._seen.setdefault(r, now)
                if now - first > self.timeout_s:
                    out[r] = "never sent a heartbeat"
                continue
            t = float(beat.split(":")[1])
            if now - t > self.timeout_s:
                out[r] = f"last heartbeat {now - t:.0f} s ago"
        return out

    def agree(self, step: int, poll_s: float = 0.0005) -> None:
        """Rendezvous before step ``step`` is launched: returns once every rank has arrived, raises
        :class:`RankFailure` as soon as a peer has reported a failure, or after ``timeout_s`` if one never arrives.
        A rank that failed calls :meth:`report_failure` instead of this, so the others stop with nothing in flight."""
        key = f"{self.prefix}/ready/{step}"
        self.store.add(key, 1)
        deadline = time.time() + self.timeout_s
        while True:
            if int(self.store.add(key, 0)) >= self.world:
                break
            for r in range(self.world):
                if r != self.rank:
                    reason = self._get(self._key("abort", r))
                    if reason is not None:
                        raise RankFailure(f"rank {r} reported: {reason}")
            if time.time() > deadline:
                raise RankFailure(f"not every rank arrived at step {step} within {self.timeout_s:.0f} s")
            time.sleep(poll_s)
        if step >= 2 and self.rank == 0:
            try:
                self.store.delete_key(f"{self.prefix}/ready/{step - 2}")
            except Exception:
                pass

    def check(self) -> None:
        """Raise :class:`RankFailure` if a peer failed; call between steps, with nothing in flight."""
        bad = self.failed_ranks()
        if bad:
            raise RankFailure("; ".join(f"rank {r} {why}" for r, why in sorted(bad.items())))


@dataclass
class _Fault:
    kind: str
    step: int
    rank: int
    seconds: float = 0.0


class FaultInjector:
    """``KSA_FAULT="raise@step=3,rank=1"`` | ``"exit@step=2,rank=0"`` | ``"stall@step=1,rank=1,seconds=5"``.

    Faults are injected on the host, between steps; nothing here launches a kernel."""

    def __init__(self, spec: Optional[str] = None, rank: int = 0):
        self.rank = rank
        self.faults: List[_Fault] = []
        spec = os.environ.get("KSA_FAULT", "") if spec is None else spec
        for item in filter(None, (s.strip() for s in spec.split(";"))):
            kind, _, rest = item.partition("@")
            kv = dict(p.split("=") for p in rest.split(",") if p)
            if kind not in ("raise", "exit", "stall"):
                raise ValueError(f"unknown fault kind {kind!r}")
            self.faults.append(_Fault(kind, int(kv.get("step", 0)), int(kv.get("rank", 0)), float(kv.get("seconds", 0))))

    def at_step(self, step: int) -> None:
        for f in self.faults:
            if f.step != step or f.rank != self.rank:
                continue
            if f.kind == "raise":
                raise RuntimeError(f"injected failure on rank {self.rank} at step {step}")
            if f.kind == "exit":
                os._exit(17)
            if f.kind == "stall":
                time.sleep(f.seconds)


def check_device() -> None:
    """Raise if a bounded device-side wait (peer flag, mbarrier) gave up since the last check."""
    from ..ops import _lib
    _lib.check_status()
