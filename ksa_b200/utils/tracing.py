"""Tracing helpers: NVTX ranges and device-side step timers.

The reference traces with ``torch.profiler`` only (``recipes/pretrain_kai_summary_unified.py:264-290``), which the
recipe here keeps behind ``--enable-profile``.  NVTX ranges cost nothing without a profiler attached and make the
phases of a step (data, step, checkpoint) visible in any CUDA timeline; :class:`StepTimer` gives per-step times from
CUDA events on the launching stream without synchronising the host on every step.
"""
from __future__ import annotations

import contextlib
import time
from typing import Dict, List, Optional

import torch


@contextlib.contextmanager
def nvtx_range(name: str, enabled: bool = True):
    """``with nvtx_range("step"):`` - an NVTX push/pop when CUDA is present, a no-op otherwise."""
    on = enabled and torch.cuda.is_available()
    if on:
        torch.cuda.nvtx.range_push(name)
    try:
        yield
    finally:
        if on:
            torch.cuda.nvtx.range_pop()


class StepTimer:
    """Device time of consecutive steps.  ``tick()`` records an event after each step; times are read back lazily
    (``times_ms()`` synchronises on the last event only).  On CPU it falls back to ``time.perf_counter``."""

    def __init__(self, device: Optional[torch.device] = None, keep: int = 4096):
        self.cuda = torch.cuda.is_available() and (device is None or torch.device(device).type == "cuda")
        self.keep = keep
        self._events: List["torch.cuda.Event"] = []
        self._host: List[float] = []
        self.tick()

    def tick(self) -> None:
        if self.cuda:
            ev = torch.cuda.Event(enable_timing=True)
            ev.record()
            self._events.append(ev)
            if len(self._events) > self.keep + 1:
                self._events.pop(0)
        else:
            self._host.append(time.perf_counter())
            if len(self._host) > self.keep + 1:
                self._host.pop(0)

    def times_ms(self) -> List[float]:
        if self.cuda:
            if len(self._events) < 2:
                return []
            self._events[-1].synchronize()
            return [a.elapsed_time(b) for a, b in zip(self._events[:-1], self._events[1:])]
        return [(b - a) * 1e3 for a, b in zip(self._host[:-1], self._host[1:])]

    def summary(self, skip: int = 0) -> Dict[str, float]:
        t = sorted(self.times_ms()[skip:])
        if not t:
            return {}
        return {"steps": len(t), "mean_ms": sum(t) / len(t), "median_ms": t[len(t) // 2], "min_ms": t[0], "max_ms": t[-1]}
