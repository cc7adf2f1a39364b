"""Checkpoint save / resume in the reference's layout (``muse/training/checkpoint.py:144-680``).

On disk: ``<output_dir>/global_step{N}/`` is a ``torch.distributed.checkpoint`` (DCP) directory whose logical tree is

    app.model.<reference parameter name>          fp32 master weights (e.g. ``model.layers.3.attn.q_proj.weight``)
    app.optim.state.<name>.{exp_avg,exp_avg_sq,step}   and   app.optim.param_groups
    app.training.{step_scheduler,lr_scheduler}

next to a ``latest`` text file naming the newest step directory and ``dataloader_state.pt`` (rank 0).  Parameter
names are the reference's (q/k/v and w1/w3 split out of the fused tensors), so its converter and ours read the same
files.  Independent switches choose what a resume restores (weights / optimizer / training state / dataloader), and
the step numbering continues from the directory name.

The engine keeps master weights and Adam moments as per-rank shards of flat unit buffers, cut anywhere inside a
parameter.  With more than one rank every saved tensor is a ``DTensor`` sharded by rows over the ranks (the layout of
the reference's FSDP2 state, ``muse/training/checkpoint.py:528-557``): each rank holds, copies to the host and writes
only ``1/world`` of the model and optimizer state, and a load re-shards for whatever world size reads it.  Moving
from the flat shards to row shards takes one all-gather of a unit at a time on the device (a few hundred MB,
transient); nothing of full size ever sits in host memory.
"""
from __future__ import annotations

import os
import re
import time
from pathlib import Path
from typing import Any, Dict, List, Optional

import torch
import torch.distributed as dist
import torch.distributed.checkpoint as dcp
from torch.distributed.checkpoint.api import CheckpointException
from torch.distributed.checkpoint.stateful import Stateful


def _rank() -> int:
    return dist.get_rank() if dist.is_available() and dist.is_initialized() else 0


def _world() -> int:
    return dist.get_world_size() if dist.is_available() and dist.is_initialized() else 1


def _barrier() -> None:
    if dist.is_available() and dist.is_initialized():
        dist.barrier()


def step_dir_name(step: int) -> str:
    return f"global_step{int(step)}"


def get_checkpoint_path(checkpoint_dir: str, checkpoint_id: Optional[str] = None) -> Optional[str]:
    """Resolve ``checkpoint_id`` (a step number, a directory name, or None / "latest") to a step directory."""
    root = Path(checkpoint_dir)
    if checkpoint_id in (None, "", "latest"):
        latest = root / "latest"
        if not latest.exists():
            return None
        name = latest.read_text().strip()
    else:
        name = str(checkpoint_id)
        if name.isdigit():
            name = step_dir_name(int(name))
    path = root / name
    return str(path) if path.is_dir() else None


def step_from_path(path: str) -> int:
    m = re.search(r"global_step(\d+)", str(path))
    return int(m.group(1)) if m else 0


# --------------------------------------------------------------------------------------------------- engine <-> tensors
def _gather_unit(engine, shard: torch.Tensor, unit) -> torch.Tensor:
    """Full fp32 flat buffer of ``unit`` from every rank's shard, on the engine's device."""
    if engine.world_size == 1:
        return shard
    group = getattr(engine, "group", None)
    shard = shard.to(engine.device).contiguous()      # offloaded state lives on the host
    if dist.get_backend(group) == "nccl":
        full = torch.empty(shard.numel() * engine.world_size, dtype=shard.dtype, device=shard.device)
        dist.all_gather_into_tensor(full, shard, group=group)
        return full
    parts = [torch.empty_like(shard) for _ in range(engine.world_size)]
    dist.all_gather(parts, shard, group=group)
    return torch.cat(parts)


def _sharded(engine) -> bool:
    return engine.world_size > 1 and dist.is_available() and dist.is_initialized()


def _mesh(engine):
    from torch.distributed.device_mesh import DeviceMesh
    m = getattr(engine, "_ckpt_mesh", None)
    if m is None:
        group = getattr(engine, "group", None) or dist.group.WORLD
        m = DeviceMesh.from_group(group, "cuda" if engine.device.type == "cuda" else "cpu")
        engine._ckpt_mesh = m
    return m


def _row_range(rows: int, world: int, rank: int):
    """Rows of a dim-0 sharded tensor that ``rank`` owns (torch's rule: chunks of ceil(rows / world))."""
    per = (rows + world - 1) // world
    lo = min(rows, rank * per)
    return lo, min(rows, lo + per)


def _to_dtensor(engine, full: torch.Tensor):
    """Keep this rank's rows of ``full`` (a copy) and describe the whole tensor as a row-sharded ``DTensor``."""
    from torch.distributed.tensor import DTensor, Shard
    if full.dim() == 0:
        full = full.reshape(1)
    lo, hi = _row_range(full.shape[0], engine.world_size, engine.rank)
    local = full[lo:hi].clone()
    return DTensor.from_local(local, _mesh(engine), [Shard(0)], run_check=False, shape=full.shape,
                              stride=full.contiguous().stride())


def _to_muse(engine, fused: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
    m = engine.model
    return m.muse_state_dict(fused) if hasattr(m, "muse_state_dict") else fused


def _from_muse(engine, muse: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
    m = engine.model
    return m.from_muse_state_dict(muse) if hasattr(m, "from_muse_state_dict") else muse


def engine_state_for_save(engine, with_optimizer: bool = True) -> Dict[str, Dict[str, torch.Tensor]]:
    """``{"model": {reference name: tensor}, "exp_avg": {...}, "exp_avg_sq": {...}}``.  One rank: CPU tensors.  Several
    ranks: row-sharded ``DTensor``s, each rank keeping only its rows."""
    out: Dict[str, Dict[str, torch.Tensor]] = {"model": {}, "exp_avg": {}, "exp_avg_sq": {}}
    kinds = [("model", "master")] + ([("exp_avg", "exp_avg"), ("exp_avg_sq", "exp_avg_sq")] if with_optimizer else [])
    sharded = _sharded(engine)
    if hasattr(engine, "sync_state"):
        engine.sync_state()
    for u in engine.units:
        for key, attr in kinds:
            full = _gather_unit(engine, getattr(u, attr), u)
            fused = {s.name: full[s.offset:s.offset + s.numel].view(s.shape) for s in u.slots}
            for name, t in _to_muse(engine, fused).items():
                out[key][name] = _to_dtensor(engine, t) if sharded else t.to("cpu", copy=True)
            del full, fused
    frozen = {s.name: s.param.detach().to(torch.float32) for s in getattr(engine, "frozen_slots", [])}
    for name, t in _to_muse(engine, frozen).items():     # frozen weights: saved with the model, no optimizer state
        out["model"][name] = _to_dtensor(engine, t) if sharded else t.to("cpu", copy=True)
    return out


def engine_state_template(engine, with_optimizer: bool = True) -> Dict[str, Dict[str, torch.Tensor]]:
    """The same tree as :func:`engine_state_for_save` with uninitialised storage: what a DCP load fills in."""
    out: Dict[str, Dict[str, torch.Tensor]] = {"model": {}, "exp_avg": {}, "exp_avg_sq": {}}
    sharded = _sharded(engine)

    def empty_like_muse(slots):
        fused = {s.name: torch.empty(s.shape, dtype=torch.float32, device="meta") for s in slots}
        res = {}
        for name, t in _to_muse(engine, fused).items():
            shape = t.shape if t.dim() > 0 else (1,)
            if sharded:
                from torch.distributed.tensor import DTensor, Shard
                lo, hi = _row_range(shape[0], engine.world_size, engine.rank)
                local = torch.empty((hi - lo,) + tuple(shape[1:]), dtype=torch.float32, device=engine.device)
                res[name] = DTensor.from_local(local, _mesh(engine), [Shard(0)], run_check=False, shape=torch.Size(shape),
                                               stride=torch.empty(shape, device="meta").stride())
            else:
                res[name] = torch.empty(shape, dtype=torch.float32)
        return res

    for u in engine.units:
        out["model"].update(empty_like_muse(u.slots))
        if with_optimizer:
            out["exp_avg"].update(empty_like_muse(u.slots))
            out["exp_avg_sq"].update(empty_like_muse(u.slots))
    out["model"].update(empty_like_muse(getattr(engine, "frozen_slots", [])))
    return out


def _full(t: torch.Tensor, device) -> torch.Tensor:
    """A loaded entry as a whole tensor on ``device`` (a row-sharded ``DTensor`` is all-gathered)."""
    if hasattr(t, "full_tensor"):
        t = t.full_tensor()
    return t.to(device=device, dtype=torch.float32)


def load_engine_state(engine, model_state: Optional[Dict[str, torch.Tensor]],
                      exp_avg: Optional[Dict[str, torch.Tensor]] = None,
                      exp_avg_sq: Optional[Dict[str, torch.Tensor]] = None, strict: bool = True) -> List[str]:
    """Write loaded tensors (reference names; whole tensors or row-sharded ``DTensor``s) into this rank's flat shards,
    one unit at a time; returns the fused names that the checkpoint lacked."""
    missing: List[str] = []
    dev = engine.device
    if hasattr(engine, "sync_state"):
        engine.sync_state()

    def unit_tensors(src, slots):
        """Fused tensors of ``slots`` assembled from the reference-named entries of ``src``."""
        if src is None:
            return None
        probe = {s.name: torch.empty(s.shape, device="meta") for s in slots}
        wanted = list(_to_muse(engine, probe))
        have = {k: _full(src[k], dev) for k in wanted if k in src}
        try:
            return _from_muse(engine, have)
        except KeyError:      # a fused tensor with some of its parts missing
            return {}

    with torch.no_grad():
        for u in engine.units:
            fused_m = unit_tensors(model_state, u.slots)
            fused_a, fused_b = unit_tensors(exp_avg, u.slots), unit_tensors(exp_avg_sq, u.slots)
            for s in u.slots:
                lo, hi = max(s.offset, u.shard_lo), min(s.offset + s.numel, u.shard_hi)
                for src, dst in ((fused_m, u.master), (fused_a, u.exp_avg), (fused_b, u.exp_avg_sq)):
                    if src is None:
                        continue
                    if s.name not in src:
                        if src is fused_m:
                            missing.append(s.name)
                        continue
                    t = src[s.name]
                    if t.numel() != s.numel:
                        raise ValueError(f"{s.name}: checkpoint shape {tuple(t.shape)} != model shape {tuple(s.shape)}")
                    if hi > lo:
                        dst[lo - u.shard_lo:hi - u.shard_lo].copy_(t.reshape(-1)[lo - s.offset:hi - s.offset])
                if fused_m is not None and s.name in fused_m:
                    u.compute[s.offset:s.offset + s.numel].copy_(fused_m[s.name].reshape(-1))
            del fused_m, fused_a, fused_b
        frozen = getattr(engine, "frozen_slots", [])
        fused_f = unit_tensors(model_state, frozen) if frozen else None
        for s in frozen:
            if fused_f is None:
                continue
            if s.name not in fused_f:
                missing.append(s.name)
                continue
            s.param.data.copy_(fused_f[s.name].view(s.shape))
    if hasattr(engine, "after_weights_loaded"):
        engine.after_weights_loaded()
    if strict and missing:
        raise KeyError(f"checkpoint lacks {len(missing)} parameters, e.g. {missing[:4]}")
    return missing


class AppState(Stateful):
    """What one checkpoint holds: model + optimizer (through the engine) and training-loop state."""

    def __init__(self, engine, step_scheduler=None, lr_scheduler=None, skip_optimizer: bool = False,
                 skip_training_state: bool = False, strict: bool = True, skip_training_state_keys=None,
                 required_training_state_keys=None, extra_training_state: Optional[Dict[str, Any]] = None):
        """``skip_training_state_keys`` / ``required_training_state_keys``: entries of the training state
        (``"step_scheduler"``, ``"lr_scheduler"``, ``"engine_step"``, names of ``extra_training_state``) that are not
        restored on load / that must be in the checkpoint (``muse/training/checkpoint.py:469-530``).
        ``extra_training_state``: further objects (with ``state_dict`` / ``load_state_dict``) or plain values saved
        under their names; restored values are available in the same dict after a load (the loading side has to list
        the names it wants, with any placeholder value: a DCP load fills the structure it is given)."""
        self.engine = engine
        self.step_scheduler = step_scheduler
        self.lr_scheduler = lr_scheduler
        self.skip_optimizer = skip_optimizer
        self.skip_training_state = skip_training_state
        self.strict = strict
        self.skip_training_state_keys = set(skip_training_state_keys or [])
        self.required_training_state_keys = set(required_training_state_keys or [])
        self.extra_training_state = extra_training_state if extra_training_state is not None else {}

    def state_dict(self) -> Dict[str, Any]:
        return self._tree(engine_state_for_save(self.engine, with_optimizer=True))

    def template(self) -> Dict[str, Any]:
        """The tree of :meth:`state_dict` with uninitialised tensors, for a load to fill (nothing is gathered)."""
        return self._tree(engine_state_template(self.engine, with_optimizer=not self.skip_optimizer))

    def _tree(self, full) -> Dict[str, Any]:
        model, m1, m2 = full["model"], full["exp_avg"], full["exp_avg_sq"]
        step = torch.tensor(float(self.engine.step_count))
        optim_state = {k: {"exp_avg": m1[k], "exp_avg_sq": m2[k], "step": step.clone()} for k in model if k in m1}
        e = self.engine
        optim = {"state": optim_state,
                 "param_groups": [{"lr": e.base_lr, "betas": (e.beta1, e.beta2), "eps": e.eps,
                                   "weight_decay": e.weight_decay, "params": list(optim_state)}]}
        training: Dict[str, Any] = {"engine_step": e.step_count}
        if self.step_scheduler is not None:
            training["step_scheduler"] = self.step_scheduler.state_dict()
        if self.lr_scheduler is not None and hasattr(self.lr_scheduler, "state_dict"):
            training["lr_scheduler"] = self.lr_scheduler.state_dict()
        for k, v in self.extra_training_state.items():
            training[k] = v.state_dict() if hasattr(v, "state_dict") and callable(v.state_dict) else v
        return {"model": model, "optim": optim, "training": training}

    def load_state_dict(self, state: Dict[str, Any]) -> None:
        model = state.get("model")
        ea = es = None
        if not self.skip_optimizer and "optim" in state:
            st = state["optim"]["state"]
            ea = {k: v["exp_avg"] for k, v in st.items()}
            es = {k: v["exp_avg_sq"] for k, v in st.items()}
        load_engine_state(self.engine, model, ea, es, strict=self.strict)
        training = state.get("training", {})
        skip = self.skip_training_state_keys
        if not self.skip_training_state:
            missing = sorted(self.required_training_state_keys - skip - set(training))
            if missing:
                raise KeyError(f"Missing required training state keys in checkpoint: {', '.join(missing)}")
        if not self.skip_optimizer and "engine_step" not in skip:
            self.engine.step_count = int(training.get("engine_step", self.engine.step_count))
        if not self.skip_training_state:
            if self.step_scheduler is not None and "step_scheduler" in training and "step_scheduler" not in skip:
                self.step_scheduler.load_state_dict(training["step_scheduler"])
            if (self.lr_scheduler is not None and "lr_scheduler" in training and "lr_scheduler" not in skip
                    and hasattr(self.lr_scheduler, "load_state_dict")):
                self.lr_scheduler.load_state_dict(training["lr_scheduler"])
            for k, v in training.items():
                if k in ("engine_step", "step_scheduler", "lr_scheduler") or k in skip:
                    continue
                target = self.extra_training_state.get(k)
                if hasattr(target, "load_state_dict") and callable(target.load_state_dict):
                    target.load_state_dict(v)
                else:
                    self.extra_training_state[k] = v


class DistributedCheckpointer:
    """DCP save (sync or async) and load of ``{"app": AppState}``."""

    def __init__(self, thread_count: int = 4, async_save: bool = False):
        self.thread_count = thread_count
        self.use_async = async_save
        self._pending = None

    def wait(self) -> None:
        if self._pending is not None:
            self._pending.result()
            self._pending = None

    def save(self, app_state: AppState, path: str) -> None:
        self.wait()
        state = {"app": app_state.state_dict()}   # materialised now so that training may go on during an async save
        writer = dcp.FileSystemWriter(path, thread_count=self.thread_count)
        if self.use_async and dist.is_available() and dist.is_initialized():
            self._pending = dcp.async_save(state, storage_writer=writer)
        else:
            dcp.save(state, storage_writer=writer, no_dist=not (dist.is_available() and dist.is_initialized()))

    def load(self, app_state: AppState, path: str) -> None:
        template = {"app": app_state.template()}
        if app_state.skip_optimizer:
            template["app"].pop("optim", None)
        dcp.load(template, storage_reader=dcp.FileSystemReader(path),
                 no_dist=not (dist.is_available() and dist.is_initialized()))
        app_state.load_state_dict(template["app"])


def save_checkpoint(app_state: AppState, checkpointer: DistributedCheckpointer, output_dir: str, step: int) -> str:
    """Write ``global_step{step}``, then point ``latest`` at it (rank 0), with barriers around the collective save."""
    path = os.path.join(output_dir, step_dir_name(step))
    if _rank() == 0:
        os.makedirs(path, exist_ok=True)
    _barrier()
    checkpointer.save(app_state, path)
    _barrier()
    if _rank() == 0:
        tmp = os.path.join(output_dir, "latest.tmp")
        with open(tmp, "w") as f:
            f.write(step_dir_name(step))
        os.replace(tmp, os.path.join(output_dir, "latest"))
    return path


def list_complete_checkpoints(checkpoint_dir: str) -> List[str]:
    """Step directories that hold a finished DCP checkpoint (the ``.metadata`` file is written last), newest first."""
    root = Path(checkpoint_dir)
    if not root.is_dir():
        return []
    steps = [p for p in root.iterdir() if p.is_dir() and re.fullmatch(r"global_step\d+", p.name)
             and (p / ".metadata").exists()]
    return [str(p) for p in sorted(steps, key=lambda p: step_from_path(p.name), reverse=True)]


def load_checkpoint(app_state: AppState, checkpointer: DistributedCheckpointer, checkpoint_dir: str,
                    checkpoint_id: Optional[str] = None, fallback: bool = False) -> Optional[int]:
    """Load ``checkpoint_id`` (default: ``latest``).  With ``fallback`` a checkpoint that is missing, unfinished or
    unreadable (a crash during the save, a damaged shard) is skipped in favour of the newest older complete one; the
    choice is a function of the directory contents only, so every rank takes the same path."""
    path = get_checkpoint_path(checkpoint_dir, checkpoint_id)
    candidates = [path] if path is not None else []
    if fallback:
        first = step_from_path(path) if path is not None else None
        candidates = [p for p in candidates if os.path.exists(os.path.join(p, ".metadata"))]
        candidates += [p for p in list_complete_checkpoints(checkpoint_dir)
                       if p not in candidates and (first is None or step_from_path(p) < first)]
    last_error: Optional[BaseException] = None
    for cand in candidates:
        try:
            checkpointer.load(app_state, cand)
            return step_from_path(cand)
        except (Exception, CheckpointException) as e:  # CheckpointException derives from BaseException
            if not fallback:
                raise
            print(f"[checkpoint] cannot load {cand}: {type(e).__name__}: {e}; trying an older one")
            last_error = e
    if last_error is not None:
        raise last_error
    return None


def save_dataloader_state(dataset, output_dir: str, step: int) -> Optional[str]:
    """Rank 0 writes the dataset's resumable state next to the step's checkpoint."""
    if not hasattr(dataset, "state_dict"):
        return None
    path = os.path.join(output_dir, step_dir_name(step), "dataloader_state.pt")
    if _rank() == 0:
        os.makedirs(os.path.dirname(path), exist_ok=True)
        torch.save(dataset.state_dict(), path)
    _barrier()
    return path


def load_dataloader_state(dataset, checkpoint_path: str) -> bool:
    """Soft resume: returns False (and leaves the dataset untouched) when there is no usable state file."""
    path = os.path.join(checkpoint_path, "dataloader_state.pt")
    if not os.path.exists(path) or not hasattr(dataset, "load_state_dict"):
        return False
    try:
        state = torch.load(path, map_location="cpu", weights_only=False)
        dataset.load_state_dict(state)
        return True
    except Exception as e:  # noqa: BLE001 - a truncated or foreign file must not kill a resume
        print(f"[checkpoint] ignoring dataloader state {path}: {type(e).__name__}: {e}")
        return False


def load_hf_checkpoint(model_dir: str, device: str = "cpu") -> Dict[str, torch.Tensor]:
    """Every tensor of an HF directory (sharded safetensors or ``pytorch_model*.bin``)."""
    from ..models.base import load_hf_state_dict
    return load_hf_state_dict(model_dir, device)


def dcp_to_state_dict(path: str) -> Dict[str, Any]:
    """Read a whole DCP directory in one process without a process group (for the converters)."""
    from torch.distributed.checkpoint.state_dict_loader import _load_state_dict
    from torch.distributed.checkpoint.default_planner import _EmptyStateDictLoadPlanner
    sd: Dict[str, Any] = {}
    _load_state_dict(sd, storage_reader=dcp.FileSystemReader(path), planner=_EmptyStateDictLoadPlanner(), no_dist=True)
    return sd
