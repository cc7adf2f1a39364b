"""Optimizer state in host memory: fp32 master weights and Adam moments live in pinned host buffers and pass through
a two-slot staging ring on the GPU while their unit is being updated.

The reference offloads parameters, gradients and optimizer state of every FSDP unit to the host and runs AdamW there
(``CPUOffloadPolicy``, muse/training/distributed.py:236-249; ``--cpu-offload`` in
recipes/pretrain_kai_summary_unified.py).  On a B200 the bf16 weights and the fp32 gradient buffer are what the
step's kernels read and write, so they stay in HBM; what leaves is the state that only the optimizer touches: 12 of
the 18 bytes per parameter that a rank's shard costs.  The update itself stays the fused kernel on the GPU
(reduce-scatter + clip + AdamW + bf16 refresh): unit ``i`` is updated from staging slot ``i % 2`` while the copy
engines bring unit ``i - 1`` in and write unit ``i + 1`` back, both under the backward pass that is still running.

Streams and events (CUDA): one stream per copy direction.  A slot is loaded only after the write-back of its last
tenant has finished (``_written``), the update waits for its load (``_loaded``), the write-back waits for the update.
All write-backs share one in-order stream, so "the last write-back of this slot is done" also covers the earlier
write-back of the unit that is being loaded again one step later.  On a CPU device (tests) the same calls run as
plain synchronous copies.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import torch

__all__ = ["OptimizerStateOffload", "host_state"]


def host_state(n: int, device: torch.device) -> torch.Tensor:
    """A zeroed ``[3, n]`` fp32 host buffer (master, exp_avg, exp_avg_sq), page-locked when ``device`` is a GPU."""
    pinned = torch.device(device).type == "cuda"
    return torch.zeros(3, max(n, 1), dtype=torch.float32, pin_memory=pinned)


class OptimizerStateOffload:
    """Staging ring for units whose ``[3, n]`` state tensor lives on the host."""

    def __init__(self, device: torch.device, max_elems: int, slots: int = 2):
        self.device = torch.device(device)
        self.cuda = self.device.type == "cuda"
        self.slots = max(int(slots), 1)
        self.staging = torch.zeros(self.slots, 3, max(max_elems, 1), dtype=torch.float32, device=self.device)
        self._tenant: List[Optional[int]] = [None] * self.slots      # unit index whose state the slot holds
        self._busy: List[bool] = [False] * self.slots                # acquired and not yet released
        self._loaded: Dict[int, "torch.cuda.Event"] = {}            # unit index -> its load has been issued
        self._written: List[Optional["torch.cuda.Event"]] = [None] * self.slots
        self.h2d_bytes = 0
        self.d2h_bytes = 0
        if self.cuda:
            self.h2d = torch.cuda.Stream(device=self.device)
            self.d2h = torch.cuda.Stream(device=self.device)

    def _slot(self, idx: int) -> int:
        return idx % self.slots

    def _view(self, idx: int, host: torch.Tensor) -> torch.Tensor:
        return self.staging[self._slot(idx), :, :host.shape[1]]

    def prefetch(self, idx: int, host: torch.Tensor) -> None:
        """Start loading unit ``idx``; a no-op if its load is already under way."""
        slot = self._slot(idx)
        if self._tenant[slot] == idx:
            return
        if self._busy[slot]:
            return      # the slot's tenant is being updated (a one-slot ring): acquire() loads the unit later
        self._tenant[slot] = idx
        dst = self._view(idx, host)
        self.h2d_bytes += host.numel() * 4
        if not self.cuda:
            dst.copy_(host)
            return
        if self._written[slot] is not None:
            self.h2d.wait_event(self._written[slot])
        with torch.cuda.stream(self.h2d):
            dst.copy_(host, non_blocking=True)
            ev = torch.cuda.Event()
            ev.record(self.h2d)
        self._loaded[idx] = ev

    def acquire(self, idx: int, host: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
        """Device views (master, exp_avg, exp_avg_sq) of unit ``idx``; the current stream waits for the load."""
        self.prefetch(idx, host)
        if self._tenant[self._slot(idx)] != idx:
            raise RuntimeError(f"unit {idx} needs the staging slot that unit {self._tenant[self._slot(idx)]} still holds")
        self._busy[self._slot(idx)] = True
        if self.cuda:
            ev = self._loaded.pop(idx, None)
            if ev is not None:
                torch.cuda.current_stream(self.device).wait_event(ev)
        v = self._view(idx, host)
        return v[0], v[1], v[2]

    def release(self, idx: int, host: torch.Tensor) -> None:
        """Write unit ``idx`` back behind the work of the current stream and give its slot up."""
        slot = self._slot(idx)
        src = self._view(idx, host)
        self.d2h_bytes += host.numel() * 4
        self._tenant[slot] = None
        self._busy[slot] = False
        if not self.cuda:
            host.copy_(src)
            return
        done = torch.cuda.Event()
        done.record(torch.cuda.current_stream(self.device))
        self.d2h.wait_event(done)
        with torch.cuda.stream(self.d2h):
            host.copy_(src, non_blocking=True)
            ev = torch.cuda.Event()
            ev.record(self.d2h)
        self._written[slot] = ev

    def synchronize(self) -> None:
        """Every write-back issued so far has reached host memory (call before the host reads or writes the state)."""
        if self.cuda:
            self.d2h.synchronize()
            self.h2d.synchronize()
        self._tenant = [None] * self.slots
        self._busy = [False] * self.slots
        self._loaded = {}
