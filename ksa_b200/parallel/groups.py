"""Process groups for data / context / tensor parallelism and the context-parallel primitives.

Grouping follows ``muse/training/parallel.py:73-133``: context-parallel (CP) groups are contiguous blocks of
``cp_size`` ranks, data-parallel (DP) groups are strided across them (``dp_size = world // cp_size``), and data is
identical within a CP group.  On top of that: Ulysses sequence<->head all-to-all (``all_to_all_4D`` and the autograd
``SeqAllToAll4D``, ``parallel.py:211-335``), an autograd all-gather (``:337-403``), batch broadcast within the CP group and
the label-preshifting CP batch split (``:148-199``).  These run on any backend (gloo on CPU in the tests, NCCL on GPUs).
"""
from __future__ import annotations

import datetime
import os
from typing import Dict, List, Optional

import torch
import torch.distributed as dist

_STATE: Dict[str, object] = {"cp_group": None, "dp_group": None, "cp_size": 1, "cp_rank": 0, "dp_rank": 0,
                             "dp_size": 1, "cp_ranks": None}
DEFAULT_TIMEOUT = datetime.timedelta(minutes=30)


def initialize_model_parallel(context_parallel_size: int = 1, timeout: datetime.timedelta = DEFAULT_TIMEOUT) -> None:
    world, rank = dist.get_world_size(), dist.get_rank()
    cp = int(context_parallel_size)
    if world % cp:
        raise ValueError(f"world size {world} is not divisible by context_parallel_size {cp}")
    dp = world // cp
    for i in range(dp):
        ranks = list(range(i * cp, (i + 1) * cp))
        g = dist.new_group(ranks, timeout=timeout)
        if rank in ranks:
            _STATE.update(cp_group=g, cp_rank=ranks.index(rank), cp_ranks=ranks)
    for j in range(cp):
        ranks = list(range(j, world, cp))
        g = dist.new_group(ranks, timeout=timeout)
        if rank in ranks:
            _STATE.update(dp_group=g, dp_rank=ranks.index(rank))
    _STATE.update(cp_size=cp, dp_size=dp)


def local_world_size(world_size: Optional[int] = None) -> int:
    """Ranks of this job on this node, from the launcher's environment (``torchrun``: ``LOCAL_WORLD_SIZE``; Open MPI,
    which the reference launches with: ``OMPI_COMM_WORLD_LOCAL_SIZE``); the whole job when neither is set or when the
    launcher's world size is not this job's."""
    e = os.environ
    env_world = int(e.get("WORLD_SIZE", e.get("OMPI_COMM_WORLD_SIZE", "0")) or 0)
    if world_size is None:
        world_size = max(env_world, 1)
    v = e.get("LOCAL_WORLD_SIZE", e.get("OMPI_COMM_WORLD_LOCAL_SIZE"))
    if not v or env_world != world_size:
        return world_size       # no launcher, or its variables describe another job (ranks spawned by hand)
    return max(1, min(int(v), world_size))


def spans_nodes(world_size: Optional[int] = None) -> bool:
    """True when the job runs on more than one node.  Peer memory (CUDA IPC over NVLink) ends at the node: the fused
    FSDP back end and the fused context-parallel exchange need their ranks on one node, across nodes the engines use
    NCCL collectives."""
    e = os.environ
    if world_size is None:
        world_size = int(e.get("WORLD_SIZE", e.get("OMPI_COMM_WORLD_SIZE", "1")))
    return local_world_size(world_size) < world_size


def check_context_parallel_placement(context_parallel_size: int, world_size: Optional[int] = None) -> None:
    """Context-parallel groups are blocks of consecutive ranks; a block must not straddle two nodes."""
    local = local_world_size(world_size)
    if context_parallel_size > 1 and (context_parallel_size > local or local % context_parallel_size):
        raise ValueError(f"context parallel size {context_parallel_size} does not fit the {local} ranks of a node: "
                         "its groups exchange keys through peer memory and must stay inside one node")


def destroy_model_parallel() -> None:
    _STATE.update(cp_group=None, dp_group=None, cp_size=1, cp_rank=0, dp_rank=0, dp_size=1, cp_ranks=None)


def get_context_parallel_group():
    return _STATE["cp_group"]


def get_data_parallel_group():
    return _STATE["dp_group"]


def get_context_parallel_world_size() -> int:
    return int(_STATE["cp_size"])


def get_context_parallel_rank() -> int:
    return int(_STATE["cp_rank"])


def get_data_parallel_world_size() -> int:
    return int(_STATE["dp_size"])


def get_data_parallel_rank() -> int:
    return int(_STATE["dp_rank"])


def get_context_parallel_ranks() -> Optional[List[int]]:
    return _STATE["cp_ranks"]


# ---------------------------------------------------------------------------- batch handling
def broadcast_batch_tensors(batch: dict, group=None, src_in_group: int = 0) -> None:
    """Make every tensor of ``batch`` equal to the CP group's first rank's (data loaders differ per rank)."""
    group = group if group is not None else get_context_parallel_group()
    if group is None or dist.get_world_size(group) == 1:
        return
    src = dist.get_global_rank(group, src_in_group)
    for k in sorted(batch):
        v = batch[k]
        if torch.is_tensor(v):
            dist.broadcast(v, src=src, group=group)


def split_batch_for_context_parallel(batch: dict, cp_rank: int, cp_size: int, ignore_index: int = -100) -> dict:
    """Create shifted labels on the full sequence, then keep this rank's contiguous slice of every per-token tensor."""
    ids = batch["input_ids"]
    mask = batch.get("loss_mask")
    if mask is None:
        mask = torch.ones_like(ids)
    shifted = torch.nn.functional.pad(ids[:, 1:], (0, 1), value=0)
    smask = torch.nn.functional.pad(mask[:, 1:], (0, 1), value=0)
    batch["labels"] = shifted * smask + ignore_index * (1 - smask)
    batch["loss_mask"] = smask
    if cp_size > 1:
        L = ids.shape[1]
        if L % cp_size:
            raise ValueError(f"sequence length {L} is not divisible by the context-parallel size {cp_size}")
        n = L // cp_size
        sl = slice(cp_rank * n, (cp_rank + 1) * n)
        for k in ("input_ids", "labels", "loss_mask", "position_ids"):
            if batch.get(k) is not None:
                batch[k] = batch[k][:, sl].contiguous()
    return batch


# ---------------------------------------------------------------------------- Ulysses all-to-all
def all_to_all_4D(x: torch.Tensor, scatter_idx: int = 2, gather_idx: int = 1, group=None) -> torch.Tensor:
    """Sequence-sharded ``[B, S/P, H, D]`` <-> head-sharded ``[B, S, H/P, D]`` (DeepSpeed-Ulysses).

    ``scatter_idx=2, gather_idx=1``: scatter heads, gather sequence; ``scatter_idx=1, gather_idx=2``: the inverse.
    """
    P = dist.get_world_size(group) if group is not None else 1
    if P == 1:
        return x
    B, s, h, d = x.shape
    if scatter_idx == 2 and gather_idx == 1:
        if h % P:
            raise ValueError(f"{h} heads cannot be split over {P} ranks")
        t = x.reshape(B, s, P, h // P, d).permute(2, 1, 0, 3, 4).contiguous()      # [P, s, B, h/P, d]
        out = torch.empty_like(t)
        dist.all_to_all_single(out, t, group=group)
        return out.reshape(P * s, B, h // P, d).transpose(0, 1).contiguous()       # [B, S, h/P, d]
    if scatter_idx == 1 and gather_idx == 2:
        if s % P:
            raise ValueError(f"sequence {s} cannot be split over {P} ranks")
        t = x.reshape(B, P, s // P, h, d).permute(1, 3, 2, 0, 4).contiguous()      # [P, h, s/P, B, d]
        out = torch.empty_like(t)
        dist.all_to_all_single(out, t, group=group)
        return out.reshape(P * h, s // P, B, d).permute(2, 1, 0, 3).contiguous()   # [B, s/P, P*h, d]
    raise ValueError("scatter_idx/gather_idx must be (2, 1) or (1, 2)")


class SeqAllToAll4D(torch.autograd.Function):
    @staticmethod
    def forward(ctx, group, x, scatter_idx, gather_idx):
        ctx.group, ctx.scatter_idx, ctx.gather_idx = group, scatter_idx, gather_idx
        return all_to_all_4D(x, scatter_idx, gather_idx, group)

    @staticmethod
    def backward(ctx, grad):
        return None, all_to_all_4D(grad.contiguous(), ctx.gather_idx, ctx.scatter_idx, ctx.group), None, None


class AllGather(torch.autograd.Function):
    """All-gather along ``dim`` whose backward returns this rank's slice of the (summed) gradient."""

    @staticmethod
    def forward(ctx, x, dim, group):
        ctx.dim, ctx.group = dim, group
        P = dist.get_world_size(group)
        parts = [torch.empty_like(x) for _ in range(P)]
        dist.all_gather(parts, x.contiguous(), group=group)
        return torch.cat(parts, dim=dim)

    @staticmethod
    def backward(ctx, grad):
        P, r = dist.get_world_size(ctx.group), dist.get_rank(ctx.group)
        grad = grad.contiguous()
        dist.all_reduce(grad, group=ctx.group)
        return grad.chunk(P, dim=ctx.dim)[r].contiguous(), None, None


def gather_by_group(x: torch.Tensor, group=None, dim: int = 0) -> torch.Tensor:
    P = dist.get_world_size(group)
    parts = [torch.empty_like(x) for _ in range(P)]
    dist.all_gather(parts, x.contiguous(), group=group)
    return torch.cat(parts, dim=dim)
