"""Training-loop utilities: default dtype context, gradient clipping by value, gradient norm, parameter freezing,
step scheduler (``muse/training/common.py:66-109,122-141,237-326,529-764``)."""
from __future__ import annotations

import contextlib
import csv
import fnmatch
import os
import re
from typing import Dict, Iterable, List, Optional, Union

import torch
import torch.nn as nn

_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float16": torch.float16, "fp16": torch.float16,
           "float32": torch.float32, "fp32": torch.float32}


def to_dtype(d: Union[str, torch.dtype]) -> torch.dtype:
    if isinstance(d, torch.dtype):
        return d
    if d not in _DTYPES:
        raise ValueError(f"unknown dtype {d!r}; one of {sorted(_DTYPES)}")
    return _DTYPES[d]


@contextlib.contextmanager
def set_default_dtype(dtype: Union[str, torch.dtype]):
    old = torch.get_default_dtype()
    torch.set_default_dtype(to_dtype(dtype))
    try:
        yield
    finally:
        torch.set_default_dtype(old)


def clip_grad_by_value(model: nn.Module, clip_range: Optional[float] = None) -> None:
    """Clamp every gradient element to ``[-clip_range, clip_range]`` (the reference clips by value, not norm).

    With the fused engine the clamp happens inside the AdamW kernel (``TrainEngine(clip_value=...)``); this
    function serves plain ``torch.optim`` loops."""
    if clip_range is None or clip_range <= 0:
        return
    nn.utils.clip_grad_value_([p for p in model.parameters() if p.grad is not None], clip_range)


def compute_grad_norm(params: Iterable[torch.Tensor], group=None) -> torch.Tensor:
    """L2 norm over (possibly sharded) gradients: local sum of squares, one scalar all-reduce when ``group`` is set
    (``compute_fsdp_zero2_grad_norm``, ``muse/training/common.py:273-326``)."""
    total = None
    for p in params:
        g = getattr(p, "grad", None)
        if g is None:
            continue
        s = g.detach().float().pow(2).sum()
        total = s if total is None else total + s
    if total is None:
        total = torch.zeros(())
    if group is not None or (torch.distributed.is_available() and torch.distributed.is_initialized() and group is not False):
        if torch.distributed.is_available() and torch.distributed.is_initialized():
            torch.distributed.all_reduce(total, group=group if group not in (None, False) else None)
    return total.sqrt()


def freeze_params_by_pattern(model: nn.Module, trainable_patterns: List[str]) -> Dict[str, int]:
    """Freeze everything whose name contains none of ``trainable_patterns`` (substring, glob or regex ``re:``).

    The distillation recipe trains only names containing ``summary_embedding`` / ``_summary``
    (``recipes/pretrain_kai_summary_unified.py:524-536``)."""
    def match(name: str) -> bool:
        for pat in trainable_patterns:
            if pat.startswith("re:"):
                if re.search(pat[3:], name):
                    return True
            elif any(c in pat for c in "*?["):
                if fnmatch.fnmatch(name, pat):
                    return True
            elif pat in name:
                return True
        return False
    stats = {"trainable": 0, "frozen": 0}
    for n, p in model.named_parameters():
        keep = match(n)
        p.requires_grad_(keep)
        stats["trainable" if keep else "frozen"] += p.numel()
    return stats


class GradNormLogger:
    """Per-parameter gradient norms appended to a CSV, one row per logged step (``common.py:328-446``)."""

    def __init__(self, path: str, every: int = 1, rank: int = 0):
        self.path, self.every, self.rank = path, every, rank
        self._header_written = False

    def log(self, step: int, named_grads) -> None:
        if self.rank != 0 or step % self.every:
            return
        rows = {n: float(g.detach().float().norm()) for n, g in named_grads if g is not None}
        os.makedirs(os.path.dirname(os.path.abspath(self.path)), exist_ok=True)
        with open(self.path, "a", newline="") as f:
            w = csv.writer(f)
            if not self._header_written:
                w.writerow(["step"] + list(rows))
                self._header_written = True
            w.writerow([step] + [f"{v:.6e}" for v in rows.values()])


class StepScheduler:
    """Micro-step / global-step bookkeeping with logging and checkpoint cadence."""

    def __init__(self, gradient_accumulation_steps: int = 1, logging_per_step: int = 100,
                 save_checkpoint_per_step: int = 1000, global_step: int = 0):
        if hasattr(gradient_accumulation_steps, "gradient_accumulation_steps"):  # an argparse namespace
            a = gradient_accumulation_steps
            gradient_accumulation_steps = a.gradient_accumulation_steps
            logging_per_step = a.logging_per_step
            save_checkpoint_per_step = a.save_checkpoint_per_step
            global_step = getattr(a, "global_step", 0)
        self.gradient_accumulation_steps = int(gradient_accumulation_steps)
        self.logging_per_step = int(logging_per_step)
        self.save_checkpoint_per_step = int(save_checkpoint_per_step)
        self._micro_step = 0
        self._global_step = int(global_step)

    def step(self) -> None:
        self._micro_step += 1
        if self.is_gradient_accumulation_boundary():
            self._global_step += 1

    @property
    def micro_step(self) -> int:
        return self._micro_step

    @property
    def global_step(self) -> int:
        return self._global_step

    def is_gradient_accumulation_boundary(self) -> bool:
        return self._micro_step > 0 and self._micro_step % self.gradient_accumulation_steps == 0

    def should_logging(self) -> bool:
        return (self._global_step > 0 and self.is_gradient_accumulation_boundary()
                and self._global_step % self.logging_per_step == 0)

    def should_save_checkpoint(self) -> bool:
        return (self._global_step > 0 and self.is_gradient_accumulation_boundary()
                and self.save_checkpoint_per_step > 0 and self._global_step % self.save_checkpoint_per_step == 0)

    def state_dict(self) -> Dict[str, int]:
        return {"gradient_accumulation_steps": self.gradient_accumulation_steps,
                "logging_per_step": self.logging_per_step,
                "save_checkpoint_per_step": self.save_checkpoint_per_step,
                "micro_step": self._micro_step, "global_step": self._global_step}

    def load_state_dict(self, state: Dict[str, int]) -> None:
        ga = state.get("gradient_accumulation_steps", self.gradient_accumulation_steps)
        if ga != self.gradient_accumulation_steps:
            raise ValueError(f"gradient_accumulation_steps mismatch: have {self.gradient_accumulation_steps}, "
                             f"checkpoint has {ga}")
        self._micro_step = int(state.get("micro_step", 0))
        self._global_step = int(state.get("global_step", 0))
