"""Small helpers shared by the trainer and the tools (``muse/utils/common.py:18-187``)."""
from __future__ import annotations

import os
import random
import time
from typing import Any, Dict

import numpy as np
import torch
import torch.distributed as dist


def get_rank() -> int:
    if dist.is_available() and dist.is_initialized():
        return dist.get_rank()
    return int(os.environ.get("RANK", os.environ.get("OMPI_COMM_WORLD_RANK", "0")))


def get_world_size() -> int:
    if dist.is_available() and dist.is_initialized():
        return dist.get_world_size()
    return int(os.environ.get("WORLD_SIZE", os.environ.get("OMPI_COMM_WORLD_SIZE", "1")))


def get_local_rank() -> int:
    return int(os.environ.get("LOCAL_RANK", os.environ.get("OMPI_COMM_WORLD_LOCAL_RANK", "0")))


def print_rank_0(*args, **kwargs) -> None:
    if get_rank() == 0:
        print(*args, **kwargs, flush=True)


def to_cuda(obj: Any, device=None, non_blocking: bool = True) -> Any:
    """Move every tensor of a (nested) container to the GPU; everything else is returned as it is."""
    if torch.is_tensor(obj):
        return obj.to(device or "cuda", non_blocking=non_blocking)
    if isinstance(obj, dict):
        return {k: to_cuda(v, device, non_blocking) for k, v in obj.items()}
    if isinstance(obj, (list, tuple)):
        return type(obj)(to_cuda(v, device, non_blocking) for v in obj)
    return obj


def set_random_seed(seed: int, deterministic: bool = False) -> None:
    random.seed(seed)
    np.random.seed(seed % (2 ** 32))
    torch.manual_seed(seed)
    if torch.cuda.is_available():
        torch.cuda.manual_seed_all(seed)
    if deterministic:
        torch.backends.cudnn.deterministic = True
        torch.backends.cudnn.benchmark = False


def dist_reduce_dict(values: Dict[str, float], op: str = "mean", group=None) -> Dict[str, float]:
    """Reduce a dict of scalars across ranks with ONE tensor all-reduce (the reference pickles the dict through
    ``all_gather_object``, ``muse/utils/common.py:57-58``).  Keys must be the same on every rank."""
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size(group) == 1:
        return dict(values)
    keys = sorted(values)
    dev = "cuda" if dist.get_backend(group) == "nccl" else "cpu"
    t = torch.tensor([float(values[k]) for k in keys], dtype=torch.float64, device=dev)
    dist.all_reduce(t, group=group)
    if op == "mean":
        t /= dist.get_world_size(group)
    return {k: float(v) for k, v in zip(keys, t.tolist())}


class Timer:
    """``with Timer("load"):`` prints the wall-clock time of the block on rank 0."""

    def __init__(self, name: str = "", verbose: bool = True):
        self.name, self.verbose, self.elapsed = name, verbose, 0.0

    def __enter__(self):
        self._t0 = time.perf_counter()
        return self

    def __exit__(self, *exc):
        self.elapsed = time.perf_counter() - self._t0
        if self.verbose:
            print_rank_0(f"[Timer] {self.name}: {self.elapsed:.3f} s")
        return False
