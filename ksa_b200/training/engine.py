"""Training engine: flat parameter storage, fp32 master weights, fused AdamW, CUDA-graph step.

The reference trains with FSDP2 ``fully_shard`` per decoder layer, bf16 compute parameters with fp32
master copies and fp32 gradient reduction, ``torch.optim.AdamW`` on the sharded fp32 tensors and
gradient clipping by value (``muse/training/distributed.py:232-287``,
``recipes/pretrain_kai_summary_unified.py:592-600,1045-1053``).  This engine owns the same state in a
layout chosen for the kernels:

* one *unit* per decoder layer plus a root unit (embeddings, final norm, head), as the reference's
  FSDP units; every unit has four flat buffers: compute weights (bf16 on GPU), fp32 master weights,
  Adam moments, and an fp32 gradient buffer;
* every ``nn.Parameter`` becomes a view of its unit's compute buffer and gets a ``main_grad`` view of
  the gradient buffer, so backward kernels write weight gradients in fp32 directly (first write of an
  accumulation window overwrites, later ones accumulate; no zero-fill pass);
* the optimizer is one fused kernel launch per unit over the flat buffers (AdamW, clip-by-value,
  bf16 refresh of the compute weights, sum of squared gradients for the grad-norm metric);
* learning rate and bias corrections live in a small device tensor, so a whole
  forward + backward + optimizer step can be captured once as a CUDA graph and replayed.

Data-parallel / FSDP sharding of these units over ranks is layered on top by
``ksa_b200.parallel.fsdp`` (which replaces ``_reduce_and_update``).
"""
from __future__ import annotations

import contextlib
import math
import os
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Sequence, Tuple

import torch
import torch.nn as nn

from .. import ops

_ALIGN = 128  # elements; keeps every parameter view 256-byte aligned in bf16 (TMA wants 16 bytes)


def _round_up(n: int, a: int) -> int:
    return (n + a - 1) // a * a


@dataclass
class ParamSlot:
    name: str
    param: nn.Parameter
    offset: int
    numel: int
    shape: torch.Size


@dataclass
class Unit:
    """One FSDP unit: flat buffers + the parameters that live in them."""
    name: str
    slots: List[ParamSlot] = field(default_factory=list)
    index: int = 0                           # position in the engine's unit list
    size: int = 0
    compute: Optional[torch.Tensor] = None   # param_dtype, full size
    master: Optional[torch.Tensor] = None    # fp32 (full, or this rank's shard under FSDP)
    exp_avg: Optional[torch.Tensor] = None
    exp_avg_sq: Optional[torch.Tensor] = None
    host_state: Optional[torch.Tensor] = None   # [3, shard] pinned host buffer behind the three views above (offload)
    grad: Optional[torch.Tensor] = None      # fp32, full size
    shard_lo: int = 0                        # [shard_lo, shard_hi): range of the flat buffer owned by this rank
    shard_hi: int = 0


class _UnitBoundary(torch.autograd.Function):
    """Identity on a layer's inputs.  Its backward runs once every backward kernel of that layer (and of everything
    after it) has been launched, and tells the engine that the unit's gradients are complete."""

    @staticmethod
    def forward(ctx, engine, tag, x, delta):
        ctx.engine, ctx.tag = engine, tag
        ctx.has_delta = delta is not None
        return (x.view_as(x), delta.view_as(delta)) if delta is not None else (x.view_as(x), None)

    @staticmethod
    def backward(ctx, gx, gd):
        ctx.engine._unit_backward_done(ctx.tag)
        return None, None, gx, (gd if ctx.has_delta else None)


class TrainEngine:
    # the single-GPU engine can update a unit on a side stream while the backward pass of the earlier units still
    # runs (the sharded engine has its own schedule and switches this off)
    _overlap_capable = True

    def __init__(self, model: nn.Module, lr: float = 4e-4, betas: Tuple[float, float] = (0.9, 0.95),
                 eps: float = 1e-8, weight_decay: float = 0.1, clip_value: float = 0.0,
                 param_dtype: Optional[torch.dtype] = None, device: Optional[torch.device] = None,
                 lr_lambda: Optional[Callable[[int], float]] = None, grad_accum_steps: int = 1,
                 world_size: int = 1, rank: int = 0, cpu_offload: bool = False,
                 overlap_optimizer: Optional[bool] = None):
        self.model = model
        self.cpu_offload = bool(cpu_offload)   # master weights and moments in pinned host memory (training/offload.py)
        self._offload = None
        self.base_lr = lr
        self.beta1, self.beta2 = betas
        self.eps, self.weight_decay, self.clip_value = eps, weight_decay, clip_value
        self.lr_lambda = lr_lambda
        self.grad_accum_steps = grad_accum_steps
        self.world_size, self.rank = world_size, rank
        self.device = torch.device(device) if device is not None else next(model.parameters()).device
        self.param_dtype = param_dtype or (torch.bfloat16 if self.device.type == "cuda" else torch.float32)
        self.step_count = 0          # optimizer steps taken
        self.micro_step = 0          # micro-batches seen in the current accumulation window
        self.units: List[Unit] = []
        self._build_units()
        self.hyper = torch.zeros(4, dtype=torch.float32, device=self.device)
        # ring of pinned staging slots: the host may run several (graph-replayed) steps ahead of the device,
        # so a slot is reused only after the copy that read it has completed
        self._hyper_ring = torch.zeros(32, 4, dtype=torch.float32)
        self._hyper_events: List[Optional[torch.cuda.Event]] = [None] * 32
        self._hyper_slot = 0
        if self.device.type == "cuda":
            self._hyper_ring = self._hyper_ring.pin_memory()
        self.grad_sq = torch.zeros(1, dtype=torch.float32, device=self.device)
        self._graphs: Dict[tuple, "_CapturedStep"] = {}
        # AdamW of a unit under the backward pass of the units in front of it: launched on a side stream as soon as
        # the unit's backward kernels have been launched (overlap_optimizer=True or KSA_OVERLAP_OPTIMIZER=1).  With
        # the state resident in HBM it measured 114.1 against 114.6 ms per step (Qwen3-1.9B-KSA, 8192 tokens: AdamW
        # and the backward GEMMs compete for the same HBM), so it is off by default there; with the state offloaded
        # to the host it hides the backward pass under the PCIe copies and is on.
        if overlap_optimizer is None:
            env = os.environ.get("KSA_OVERLAP_OPTIMIZER")
            overlap_optimizer = (env == "1") if env is not None else (self.cpu_offload and self.device.type == "cuda")
        self.overlap_optimizer = bool(overlap_optimizer) and self._overlap_capable
        self._hooks_active = False
        self._overlap_step = False
        self._async_done: set = set()
        self.opt_stream = None       # CPU (tests): the update runs in place, inside the backward pass
        if self.overlap_optimizer:
            if self.device.type == "cuda":
                self.opt_stream = torch.cuda.Stream(device=self.device)
            self._install_overlap_hooks()

    # ------------------------------------------------------------------ construction
    def _unit_modules(self) -> List[Tuple[str, List[Tuple[str, nn.Parameter]]]]:
        model = self.model
        layer_mods = model.get_layers_to_shard() if hasattr(model, "get_layers_to_shard") else []
        taken = set()
        units = []
        names = {id(p): n for n, p in model.named_parameters()}
        # Frozen parameters (requires_grad False when the engine is built, e.g. the base weights of a distillation
        # run) stay out of the units: nothing decays or updates them, as in the reference, whose optimizer holds
        # only trainable parameters (muse/models/base.py:380-388).
        frozen = {id(p) for p in model.parameters() if not p.requires_grad}
        self._frozen_params = [(names[i], p) for i, p in ((id(p), p) for p in model.parameters()) if i in frozen]
        for i, m in enumerate(layer_mods):
            ps = [(names[id(p)], p) for p in m.parameters() if id(p) not in frozen]
            taken.update(id(p) for p in m.parameters())
            units.append((f"layer{i}", ps))
        # what is left is split in two: parameters used before the layers (embeddings) and after them (norm, head)
        root = [(n, p) for n, p in model.named_parameters() if id(p) not in taken and id(p) not in frozen]
        embed = [(n, p) for n, p in root if "embedding" in n]
        head = [(n, p) for n, p in root if "embedding" not in n]
        out = []
        if embed:
            out.append(("embed", embed))
        out += units
        if head:
            out.append(("head", head))
        return out

    def _shard_range(self, size: int) -> Tuple[int, int]:
        per = size // self.world_size
        return self.rank * per, (self.rank + 1) * per

    def _build_units(self) -> None:
        dev = self.device
        planned: List[Unit] = []
        for uname, ps in self._unit_modules():
            unit = Unit(uname)
            off = 0
            for n, p in ps:
                unit.slots.append(ParamSlot(n, p, off, p.numel(), p.shape))
                off += _round_up(p.numel(), _ALIGN)
            unit.size = _round_up(max(off, _ALIGN), _ALIGN * max(self.world_size, 1))
            unit.shard_lo, unit.shard_hi = self._shard_range(unit.size)
            planned.append(unit)
        self._allocate_storage(planned)
        if self.cpu_offload:
            from .offload import OptimizerStateOffload
            self._offload = OptimizerStateOffload(dev, max(u.shard_hi - u.shard_lo for u in planned))
        self._place_frozen()
        for unit in planned:
            with torch.no_grad():
                for s in unit.slots:
                    src = s.param.detach().to(device=dev, dtype=torch.float32).reshape(-1)
                    unit.compute[s.offset:s.offset + s.numel].copy_(src)
                    self._master_init(unit, s, src)
                    s.param.data = unit.compute[s.offset:s.offset + s.numel].view(s.shape)
                    s.param.main_grad = unit.grad[s.offset:s.offset + s.numel].view(s.shape)
                    s.param._grad_written = False
            unit.index = len(self.units)
            self.units.append(unit)

    def _place_frozen(self) -> None:
        """Frozen parameters: one flat buffer in the compute dtype, replicated on every rank; no master copy, no
        moments, no gradient buffer."""
        self.frozen_slots: List[ParamSlot] = []
        off = 0
        for n, p in self._frozen_params:
            self.frozen_slots.append(ParamSlot(n, p, off, p.numel(), p.shape))
            off += _round_up(p.numel(), _ALIGN)
        self.frozen_compute = torch.zeros(max(off, 1), dtype=self.param_dtype, device=self.device)
        with torch.no_grad():
            for s in self.frozen_slots:
                view = self.frozen_compute[s.offset:s.offset + s.numel].view(s.shape)
                view.copy_(s.param.detach().to(device=self.device, dtype=torch.float32))
                s.param.data = view

    def _allocate_storage(self, units: List[Unit]) -> None:
        """Allocate compute / gradient / optimizer-state buffers of every unit (overridden for symmetric memory)."""
        dev = self.device
        for unit in units:
            unit.compute = torch.zeros(unit.size, dtype=self.param_dtype, device=dev)
            unit.grad = torch.zeros(unit.size, dtype=torch.float32, device=dev)
            self._alloc_shard_state(unit)

    def _alloc_shard_state(self, unit: Unit) -> None:
        n = unit.shard_hi - unit.shard_lo
        dev = self.device
        if self.cpu_offload:
            from .offload import host_state
            unit.host_state = host_state(n, dev)
            unit.master, unit.exp_avg, unit.exp_avg_sq = (unit.host_state[i, :n] for i in range(3))
            return
        unit.master = torch.zeros(n, dtype=torch.float32, device=dev)
        unit.exp_avg = torch.zeros(n, dtype=torch.float32, device=dev)
        unit.exp_avg_sq = torch.zeros(n, dtype=torch.float32, device=dev)

    def _master_init(self, unit: Unit, s: ParamSlot, src_f32: torch.Tensor) -> None:
        lo, hi = max(s.offset, unit.shard_lo), min(s.offset + s.numel, unit.shard_hi)
        if hi > lo:
            unit.master[lo - unit.shard_lo:hi - unit.shard_lo].copy_(src_f32[lo - s.offset:hi - s.offset])

    # ------------------------------------------------------------------ schedule
    def current_lr(self, step: Optional[int] = None) -> float:
        step = self.step_count if step is None else step
        return self.base_lr * (self.lr_lambda(step) if self.lr_lambda is not None else 1.0)

    def _write_hyper(self) -> None:
        t = self.step_count + 1
        slot = self._hyper_slot
        self._hyper_slot = (slot + 1) % len(self._hyper_events)
        if self._hyper_events[slot] is not None:
            self._hyper_events[slot].synchronize()
        h = self._hyper_ring[slot]
        h[0] = self.current_lr()
        h[1] = 1.0 - self.beta1 ** t
        h[2] = 1.0 - self.beta2 ** t
        h[3] = 1.0 / (self.grad_accum_steps * max(self.world_size, 1))
        self.hyper.copy_(h, non_blocking=True)
        if self.device.type == "cuda":
            ev = torch.cuda.Event()
            ev.record(torch.cuda.current_stream(self.device))
            self._hyper_events[slot] = ev

    # ------------------------------------------------------------------ gradients
    def zero_grad(self) -> None:
        for u in self.units:
            for s in u.slots:
                s.param._grad_written = False
                s.param.grad = None

    def _collect_autograd_grads(self) -> None:
        """Fold ``.grad`` (ops without a main_grad path, the CPU path) into the fp32 buffers; zero the rest."""
        for u in self.units:
            self._collect_unit_grads(u)

    @staticmethod
    def _collect_unit_grads(u: Unit) -> None:
        for s in u.slots:
            p = s.param
            if p.grad is not None:
                if getattr(p, "_grad_written", False):
                    p.main_grad.add_(p.grad.to(torch.float32))
                else:
                    p.main_grad.copy_(p.grad)
                    p._grad_written = True
                p.grad = None
            elif not getattr(p, "_grad_written", False):
                p.main_grad.zero_()
                p._grad_written = True

    # ------------------------------------------------------------------ optimizer under the backward pass
    def _install_overlap_hooks(self) -> None:
        model = self.model
        layers = list(model.get_layers_to_shard()) if hasattr(model, "get_layers_to_shard") else []
        names = [u.name for u in self.units]
        for i, layer in enumerate(layers):
            if f"layer{i}" in names:
                layer.register_forward_pre_hook(self._make_unit_pre_hook(names.index(f"layer{i}")))
        if layers and "head" in names:
            layers[-1].register_forward_hook(self._make_head_hook(names.index("head")))

    def _make_unit_pre_hook(self, ui: int):
        def hook(module, args):
            x, delta = args[0], args[1]
            if self._hooks_active and torch.is_grad_enabled() and x.requires_grad:
                x, delta = _UnitBoundary.apply(self, ui, x, delta)
                return (x, delta) + tuple(args[2:])
            return None
        return hook

    def _make_head_hook(self, head_ui: int):
        def hook(module, args, output):
            if self._hooks_active and torch.is_grad_enabled() and isinstance(output, tuple) and output[0].requires_grad:
                return _UnitBoundary.apply(self, head_ui, output[0], output[1]) + tuple(output[2:])
            return None
        return hook

    def _unit_backward_done(self, ui: int) -> None:
        """Every backward kernel that writes unit ``ui``'s gradients has been launched: update it on the side stream."""
        if not self._hooks_active or ui in self._async_done:
            return
        u = self.units[ui]
        self._collect_unit_grads(u)
        if self.opt_stream is None:
            self._reduce_and_update(u)
        else:
            ev = torch.cuda.Event()
            ev.record(torch.cuda.current_stream(self.device))
            with torch.cuda.stream(self.opt_stream):
                self.opt_stream.wait_event(ev)
                self._reduce_and_update(u)
        self._async_done.add(ui)

    # ------------------------------------------------------------------ optimizer
    @contextlib.contextmanager
    def _optimizer_state(self, unit: Unit):
        """(master, exp_avg, exp_avg_sq) of ``unit`` as tensors on the engine's device for the duration of the block.
        With the state offloaded to the host they are views of a staging slot: loaded before the block (the current
        stream waits for the copy), written back after it, and the unit that is updated next starts loading."""
        if self._offload is None:
            yield unit.master, unit.exp_avg, unit.exp_avg_sq
            return
        idx = unit.index
        state = self._offload.acquire(idx, unit.host_state)
        if idx > 0:
            self._offload.prefetch(idx - 1, self.units[idx - 1].host_state)
        try:
            yield state
        finally:
            self._offload.release(idx, unit.host_state)

    def sync_state(self) -> None:
        """Offloaded state only: wait until every write-back has reached host memory.  Called before the host reads
        or overwrites master weights or moments (checkpoints, weight loading)."""
        if self._offload is not None:
            self._offload.synchronize()

    def _reduce_and_update(self, unit: Unit) -> None:
        """Single rank: AdamW over the whole unit.  The FSDP engine overrides this with the fused
        reduce-scatter + AdamW + weight all-gather."""
        with self._optimizer_state(unit) as (master, exp_avg, exp_avg_sq):
            ops.adamw_step(master, unit.grad, exp_avg, exp_avg_sq,
                           unit.compute if self.param_dtype != torch.float32 else None,
                           self.hyper, self.beta1, self.beta2, self.eps, self.weight_decay, self.clip_value,
                           self.grad_sq)
            if self.param_dtype == torch.float32:
                unit.compute.copy_(master)

    def optimizer_step(self) -> None:
        self._collect_autograd_grads()
        if not self._overlap_step:
            self.grad_sq.zero_()
            self._async_done = set()
        for unit in reversed(self.units):
            if unit.index not in self._async_done:     # updated under the backward pass already
                self._reduce_and_update(unit)
        if self._overlap_step and self.opt_stream is not None:
            torch.cuda.current_stream(self.device).wait_stream(self.opt_stream)
        self._overlap_step = False
        self._async_done = set()
        self._finish_step()

    def _finish_step(self) -> None:
        pass

    def grad_norm(self) -> torch.Tensor:
        """Global L2 norm of the (averaged) gradients of the last optimizer step, as a device scalar."""
        return self.grad_sq.sqrt()

    # ------------------------------------------------------------------ steps
    def forward_backward(self, tokens: torch.Tensor, labels: torch.Tensor, step_fn=None, **kw) -> torch.Tensor:
        """Forward and backward of one micro-batch.  ``step_fn(tokens, labels) -> loss`` replaces the plain language
        model loss: it must run the model's forward AND one backward pass itself and return the detached loss
        (distillation uses it), so that whatever the engine hangs on the forward and backward passes still applies."""
        self._async_done = set()
        self._overlap_step = self.overlap_optimizer and self.micro_step + 1 == self.grad_accum_steps
        self._hooks_active = self._overlap_step
        if self._overlap_step:
            self.grad_sq.zero_()        # the units add their sums of squares while the backward pass still runs
        try:
            if step_fn is not None:
                return step_fn(tokens, labels)
            loss = self.model(tokens, labels=labels, **kw)
            loss.backward()
            return loss.detach()
        finally:
            self._hooks_active = False

    def train_step(self, tokens: torch.Tensor, labels: torch.Tensor, **kw) -> torch.Tensor:
        """One micro-batch; runs the optimizer at the accumulation boundary.  Returns the loss (device)."""
        if self.micro_step == 0:
            self.zero_grad()
        if tokens.device != self.device:  # e.g. pinned host batches
            tokens = tokens.to(self.device, non_blocking=True)
            labels = labels.to(self.device, non_blocking=True)
        if self.micro_step + 1 == self.grad_accum_steps:
            self._write_hyper()     # before the backward pass: units may be updated while it still runs
        loss = self.forward_backward(tokens, labels, **kw)
        self.micro_step += 1
        if self.micro_step == self.grad_accum_steps:
            self.optimizer_step()
            self.step_count += 1
            self.micro_step = 0
        return loss

    # ------------------------------------------------------------------ CUDA-graph step
    def graphed_step(self, tokens: torch.Tensor, labels: torch.Tensor) -> torch.Tensor:
        """``train_step`` replayed from a CUDA graph captured on first use for this shape.

        ``tokens``/``labels`` may live in pinned host memory: they are copied into the graph's static
        inputs on the current stream.  Needs ``grad_accum_steps == 1`` windows to be uniform: a graph is
        keyed by (shape, first micro-step?, boundary?).
        """
        # the staging ring is driven from the host, and deterministic mode sizes a buffer from the data (a host
        # synchronisation, which a stream capture forbids): both steps stay eager
        if self._offload is not None or ops.is_deterministic():
            return self.train_step(tokens, labels)
        first = self.micro_step == 0
        boundary = self.micro_step + 1 == self.grad_accum_steps
        key = (tuple(tokens.shape), first, boundary)
        cap = self._graphs.get(key)
        if cap is None:
            cap = _CapturedStep(self, tokens.shape, first, boundary)
            self._graphs[key] = cap
        cap.tokens.copy_(tokens, non_blocking=True)
        cap.labels.copy_(labels, non_blocking=True)
        if boundary:
            self._write_hyper()
        cap.graph.replay()
        self.micro_step += 1
        if boundary:
            self.step_count += 1
            self.micro_step = 0
        return cap.loss

    # ------------------------------------------------------------------ state
    def named_master_params(self):
        """(name, fp32 tensor view) for every parameter whose master copy is fully local (single rank)."""
        self.sync_state()
        for u in self.units:
            for s in u.slots:
                if s.offset >= u.shard_lo and s.offset + s.numel <= u.shard_hi:
                    lo = s.offset - u.shard_lo
                    yield s.name, u.master[lo:lo + s.numel].view(s.shape)

    def state_dict(self) -> dict:
        self.sync_state()
        return {
            "step": self.step_count,
            "units": {u.name: {"master": u.master, "exp_avg": u.exp_avg, "exp_avg_sq": u.exp_avg_sq,
                               "shard": (u.shard_lo, u.shard_hi), "size": u.size,
                               "slots": [(s.name, s.offset, s.numel, tuple(s.shape)) for s in u.slots]}
                      for u in self.units},
        }

    def load_state_dict(self, state: dict, load_optimizer: bool = True) -> None:
        self.step_count = int(state.get("step", 0)) if load_optimizer else self.step_count
        self.sync_state()
        for u in self.units:
            su = state["units"][u.name]
            u.master.copy_(su["master"])
            if load_optimizer:
                u.exp_avg.copy_(su["exp_avg"])
                u.exp_avg_sq.copy_(su["exp_avg_sq"])
        self.refresh_compute_from_master()

    def refresh_compute_from_master(self) -> None:
        self.sync_state()
        for u in self.units:
            if self.world_size == 1:
                u.compute.copy_(u.master)

    def load_model_weights(self, state: Dict[str, torch.Tensor]) -> None:
        """Overwrite compute and master weights from a (fused-name) model state dict."""
        self.sync_state()
        with torch.no_grad():
            for u in self.units:
                for s in u.slots:
                    if s.name not in state:
                        continue
                    src = state[s.name].to(device=self.device, dtype=torch.float32).reshape(-1)
                    u.compute[s.offset:s.offset + s.numel].copy_(src)
                    self._master_init(u, s, src)
            for s in self.frozen_slots:
                if s.name in state:
                    s.param.data.copy_(state[s.name].to(device=self.device, dtype=torch.float32).view(s.shape))
        if hasattr(self, "after_weights_loaded"):
            self.after_weights_loaded()


class _CapturedStep:
    def __init__(self, engine: TrainEngine, shape, first: bool, boundary: bool, warmup: bool = True):
        dev = engine.device
        self.tokens = torch.zeros(shape, dtype=torch.long, device=dev)
        self.labels = torch.zeros(shape, dtype=torch.long, device=dev)
        if warmup:
            self._warm_up(engine, first, boundary)
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            self.loss = self._run(engine, first, boundary)

    def _warm_up(self, engine: TrainEngine, first: bool, boundary: bool) -> None:
        """One uncaptured run on a side stream (allocator pools, kernel attributes, status words), undoing its effects
        on the training state.  Engines whose step talks to other ranks warm up with a real step instead."""
        dev = engine.device
        snap = [(u.master.clone(), u.exp_avg.clone(), u.exp_avg_sq.clone(), u.compute.clone()) for u in engine.units]
        grads = None if first else [u.grad.clone() for u in engine.units]
        side = torch.cuda.Stream(device=dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):
            self._run(engine, first, boundary)
        torch.cuda.current_stream(dev).wait_stream(side)
        torch.cuda.synchronize(dev)
        for u, (ma, m, v, c) in zip(engine.units, snap):
            u.master.copy_(ma); u.exp_avg.copy_(m); u.exp_avg_sq.copy_(v); u.compute.copy_(c)
        if grads is not None:
            for u, g in zip(engine.units, grads):
                u.grad.copy_(g)
        del snap, grads

    def _run(self, engine: TrainEngine, first: bool, boundary: bool) -> torch.Tensor:
        for u in engine.units:
            for s in u.slots:
                s.param._grad_written = not first
                s.param.grad = None
        loss = engine.forward_backward(self.tokens, self.labels)
        if boundary:
            engine.optimizer_step()
        return loss
