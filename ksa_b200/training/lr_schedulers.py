"""Learning-rate schedules as pure functions of the optimizer step.

``get_lr_lambda(name, ...)`` returns ``f(step) -> multiplier`` which the training engine feeds to its
device-side hyper-parameter tensor; ``get_scheduler`` wraps the same function in a ``LambdaLR`` for code that
drives a ``torch.optim`` optimizer.  Shapes and edge cases follow ``muse/training/lr_schedulers.py:45-437``:

* ``cosine``: zero for ``num_stop_steps``, linear warm-up, cosine decay to ``min_lr_rate`` at
  ``num_training_steps``, ``min_lr_rate`` afterwards;
* ``cosine_v2``: the cosine ends at ``num_decay_steps`` and the rate is held until the end;
* ``wsd``: warm-up, stable at 1, linear decay over the last ``num_decay_steps`` steps;
* ``constant``: warm-up, then 1.
"""
from __future__ import annotations

import math
from functools import partial
from typing import Callable, Optional


def cosine_lambda(step: int, *, num_warmup_steps: int, num_training_steps: int, num_cycles: float = 0.5,
                  num_stop_steps: int = 0, min_lr_rate: float = 0.0) -> float:
    if num_stop_steps > 0 and step < num_stop_steps:
        return 0.0
    if step < num_warmup_steps:
        return step / max(1, num_warmup_steps)
    if step > num_training_steps:
        return min_lr_rate
    progress = (step - num_warmup_steps) / max(1, num_training_steps - num_warmup_steps)
    factor = 0.5 * (1.0 + math.cos(math.pi * num_cycles * 2.0 * progress))
    return max(0.0, factor * (1 - min_lr_rate) + min_lr_rate)


def cosine_v2_lambda(step: int, *, num_warmup_steps: int, num_decay_steps: int, num_training_steps: int,
                     num_cycles: float = 0.5, num_stop_steps: int = 0, min_lr_rate: float = 0.0) -> float:
    if num_stop_steps > 0 and step < num_stop_steps:
        return 0.0
    if step < num_warmup_steps:
        return step / max(1, num_warmup_steps)
    if step > num_training_steps or step > num_decay_steps:
        return min_lr_rate
    progress = (step - num_warmup_steps) / max(1, num_decay_steps - num_warmup_steps)
    factor = 0.5 * (1.0 + math.cos(math.pi * num_cycles * 2.0 * progress))
    return max(0.0, factor * (1 - min_lr_rate) + min_lr_rate)


def wsd_lambda(step: int, *, num_warmup_steps: int, num_decay_steps: int, num_training_steps: int,
               min_lr_rate: float = 0.0) -> float:
    if step < num_warmup_steps:
        return step / max(1, num_warmup_steps)
    if step >= num_training_steps:
        return min_lr_rate
    decay_start = num_training_steps - num_decay_steps
    if step < decay_start:
        return 1.0
    progress = (step - decay_start) / max(1, num_decay_steps)
    return 1.0 - progress * (1.0 - min_lr_rate)


def constant_lambda(step: int, *, num_warmup_steps: int = 0) -> float:
    if step < num_warmup_steps:
        return step / max(1, num_warmup_steps)
    return 1.0


def _min_rate(base_lr: Optional[float], min_lr: Optional[float], min_lr_rate: Optional[float]) -> float:
    if min_lr is not None and min_lr_rate is not None:
        raise ValueError("give only one of min_lr and min_lr_rate")
    if min_lr is not None:
        if not base_lr:
            raise ValueError("min_lr needs the base learning rate to become a rate")
        return min_lr / base_lr
    return 0.0 if min_lr_rate is None else min_lr_rate


def get_lr_lambda(name: str, *, num_warmup_steps: int = 0, num_training_steps: Optional[int] = None,
                  num_decay_steps: Optional[int] = None, num_cycles: float = 0.5, num_stop_steps: int = 0,
                  base_lr: Optional[float] = None, min_lr: Optional[float] = None,
                  min_lr_rate: Optional[float] = None) -> Callable[[int], float]:
    rate = _min_rate(base_lr, min_lr, min_lr_rate)
    if name == "cosine":
        return partial(cosine_lambda, num_warmup_steps=num_warmup_steps, num_training_steps=num_training_steps,
                       num_cycles=num_cycles, num_stop_steps=num_stop_steps, min_lr_rate=rate)
    if name == "cosine_v2":
        return partial(cosine_v2_lambda, num_warmup_steps=num_warmup_steps, num_decay_steps=num_decay_steps,
                       num_training_steps=num_training_steps, num_cycles=num_cycles, num_stop_steps=num_stop_steps,
                       min_lr_rate=rate)
    if name == "wsd":
        return partial(wsd_lambda, num_warmup_steps=num_warmup_steps, num_decay_steps=num_decay_steps or 0,
                       num_training_steps=num_training_steps, min_lr_rate=rate)
    if name == "constant":
        return partial(constant_lambda, num_warmup_steps=num_warmup_steps or 0)
    raise NotImplementedError(f"unsupported LR scheduler {name!r}")


def get_scheduler(name: str, optimizer, num_warmup_steps: Optional[int] = None,
                  num_training_steps: Optional[int] = None, last_epoch: int = -1, **kwargs):
    """``torch.optim.lr_scheduler.LambdaLR`` with the named schedule (``min_lr`` is absolute)."""
    from torch.optim.lr_scheduler import LambdaLR
    fn = get_lr_lambda(name, num_warmup_steps=num_warmup_steps or 0, num_training_steps=num_training_steps,
                       base_lr=optimizer.defaults["lr"], **kwargs)
    return LambdaLR(optimizer, fn, last_epoch)
