"""FSDP (ZeRO-2 style) on top of :class:`ksa_b200.training.engine.TrainEngine`.

Sharding follows the reference (``muse/training/distributed.py:232-287``): one unit per decoder layer plus the
remaining parameters (here split into an ``embed`` and a ``head`` unit), bf16 compute weights resident on every
rank (``reshard_after_forward=False``, the reference scripts' default), fp32 master weights, Adam moments and
gradient reduction in fp32, each rank owning ``1/world`` of every unit's flat buffer.

Two communication back ends behind one engine:

``comm="fused"`` (GPUs, the product path)
    Compute and gradient buffers live in symmetric memory (``ksa_b200.parallel.symm``).
    * Gradient reduce-scatter + cast/scale + AdamW is ONE kernel on the shard owner that reads every rank's fp32
      gradients over NVLink (``ksa_peer_reduce_adamw``); the parameter all-gather is a P2P pull of the peers'
      updated bf16 shards (``ksa_peer_gather``).  No NCCL collective is on the step's path.
    * ``overlap="stream"`` (default): both run on a side stream as soon as a unit's backward has been launched
      (reduce + AdamW) or one unit ahead of the forward pass (gather).  Their CTAs need almost no shared memory, so
      they are co-resident with the GEMM CTAs on the same SMs and the NVLink / HBM traffic hides under tensor work.
    * ``overlap="gemm2"``: the gather of the next unit rides inside the gate/up projection of the current layer (the
      longest forward GEMM): a communication warp in every CTA of that CTA-pair GEMM moves the peers' shards with
      bulk copies through a small shared-memory ring while the other warps compute (``ksa_gemm2_gather_bf16``).  A unit cannot be pulled inside
      its own first GEMM, because the RMSNorm in front of the QKV projection already reads the unit's scale vector.
      Reduce + AdamW stays on the side stream.
    * Cross-GPU ordering uses per-(unit, rank) flags in symmetric signal pads carrying the step number; every wait
      is bounded and reports through the library's status word.

``reshard_after_forward=True`` (ZeRO-3, fused back end with ``overlap="stream"``)
    The reference's ``fully_shard(..., reshard_after_forward=True)`` (``muse/training/distributed.py:236-287``).  Every
    rank keeps only its ``1/world`` shard of each unit's bf16 weights (symmetric memory, written by the reduce + AdamW
    kernel) plus a small pool of full-size slots: three for decoder layers, one shared by the embedding and the head.
    A unit is gathered into its slot one unit ahead of the forward pass and, if a later unit has taken the slot
    since, again one unit ahead of its backward pass (also the recomputation of a checkpointed layer); parameters keep
    fixed addresses because a unit always lives in the same slot.  Resident bf16 weights drop from the whole model to
    ``model / world + 3 layers + max(embedding, head)``.

``comm="collective"`` (any backend, incl. gloo on CPU; the NCCL baseline for A/B runs)
    ``reduce_scatter`` -> AdamW on the shard -> ``all_gather``, per unit, after backward.
"""
from __future__ import annotations

import ctypes
from typing import List, Optional

import torch
import torch.distributed as dist
import torch.nn as nn

from .. import ops
from ..ops import _lib
from ..training.engine import TrainEngine, Unit


class _Boundary(torch.autograd.Function):
    """Identity on (x, delta) whose backward reports that everything downstream of it has run its backward."""

    @staticmethod
    def forward(ctx, engine, tag, x, delta):
        ctx.engine, ctx.tag = engine, tag
        ctx.has_delta = delta is not None
        return (x.view_as(x), delta.view_as(delta)) if delta is not None else (x.view_as(x), None)

    @staticmethod
    def backward(ctx, gx, gd):
        ctx.engine._backward_residency(ctx.tag)
        ctx.engine._backward_reached(ctx.tag)
        return None, None, gx, (gd if ctx.has_delta else None)


def default_overlap(world_size: int, context_parallel: int = 1, reshard_after_forward: bool = False) -> str:
    """The overlap mode a run gets when it does not ask for one.  Measured on Qwen3-1.9B-KSA, 8192 tokens per GPU:
    ``gemm2`` (the next unit's gather inside the gate/up GEMM) against ``stream``: 127.1 / 127.7 ms per step on 2 GPUs,
    117.3 / 119.5 and 118.6 / 120.6 on 4 (two boxes), 118.8 / 121.2 on 8.  So plain data-parallel runs on 4 or more
    GPUs take ``gemm2``; context-parallel runs and ZeRO-3 storage keep ``stream`` (the only mode they ran with)."""
    if world_size >= 4 and context_parallel == 1 and not reshard_after_forward:
        return "gemm2"
    return "stream"


class FsdpEngine(TrainEngine):
    _overlap_capable = False      # this engine schedules reduce + update under the backward pass itself

    def __init__(self, model: nn.Module, *args, world_size: int = 1, rank: int = 0, group=None, comm: Optional[str] = None,
                 overlap: str = "stream", pair_gather_min_flops: float = 3e11, reshard_after_forward: bool = False,
                 **kw):
        self.group = group
        self.reshard = bool(reshard_after_forward)
        if overlap not in ("stream", "gemm2"):
            raise ValueError(f"overlap must be 'stream' or 'gemm2', not {overlap!r}")
        self.overlap = overlap
        self.pair_gather_min_flops = pair_gather_min_flops    # only a GEMM at least this long carries a gather
        dev = kw.get("device") or next(model.parameters()).device
        from .groups import spans_nodes
        # the fused back end reaches the other ranks through CUDA IPC peer memory, which ends at the node
        one_node = not spans_nodes(world_size)
        self.comm = comm or ("fused" if torch.device(dev).type == "cuda" and world_size > 1 and one_node
                             else "collective")
        if self.comm == "fused" and not one_node:
            raise ValueError("comm='fused' needs all ranks on one node (peer memory); use comm='collective' across nodes")
        if self.reshard and (self.comm != "fused" or overlap != "stream" or world_size < 2):
            raise ValueError("reshard_after_forward needs the fused back end with overlap='stream' on 2 or more ranks")
        self._slot_holds = {}          # pool slot -> unit index whose weights it holds
        self._resident_ev = {}         # unit index -> event of the gather that made it resident
        self._in_backward = False
        self._symm = []
        super().__init__(model, *args, world_size=world_size, rank=rank, **kw)
        self.epoch = torch.zeros(1, dtype=torch.int32, device=self.device)
        # Number carried by the cross-GPU flags: optimizer steps taken by THIS engine object.  It is not step_count,
        # which a checkpoint load moves forward while the flags of a fresh process still hold zero.
        self._flag_epoch = 0
        self._epoch_ring = torch.zeros(32, 1, dtype=torch.int32)
        if self.device.type == "cuda":
            self._epoch_ring = self._epoch_ring.pin_memory()
        self._grad_sq_reduced = None
        if self.comm == "fused":
            from .symm import SignalPad
            n = len(self.units) * self.world_size
            self.pad_grads = SignalPad(n, group, self.device)
            self.pad_weights = SignalPad(n, group, self.device)
            self.comm_stream = torch.cuda.Stream(device=self.device)
            self._gather_done = {}
            self._install_hooks()
            if self.reshard:
                self._shards_from_master()

    # ------------------------------------------------------------------ storage
    def _allocate_storage(self, units: List[Unit]) -> None:
        if self.comm != "fused":
            return super()._allocate_storage(units)
        if self.reshard:
            return self._allocate_resharded(units)
        from .symm import SymmetricBuffer
        item = torch.empty((), dtype=self.param_dtype).element_size()
        total = sum(u.size for u in units)
        self._sym_compute = SymmetricBuffer(total * item, self.group, self.device)
        self._sym_grad = SymmetricBuffer(total * 4, self.group, self.device)
        self._symm += [self._sym_compute, self._sym_grad]
        off = 0
        for u in units:
            u.compute = self._sym_compute.view(self.param_dtype, off * item, u.size)
            u.grad = self._sym_grad.view(torch.float32, off * 4, u.size)
            u.compute_ptrs = self._sym_compute.offset_ptr_array(off * item)
            u.grad_ptrs = self._sym_grad.offset_ptr_array(off * 4)
            self._alloc_shard_state(u)
            off += u.size

    def _allocate_resharded(self, units: List[Unit]) -> None:
        """ZeRO-3 storage: persistent bf16 shards (symmetric: the peers pull from them) and a pool of full-size slots."""
        from .symm import SymmetricBuffer
        item = torch.empty((), dtype=self.param_dtype).element_size()
        W = self.world_size
        total = sum(u.size for u in units)
        layer_units = [u for u in units if u.name.startswith("layer")]
        other_units = [u for u in units if not u.name.startswith("layer")]
        lay = max([u.size for u in layer_units], default=0)
        big = max([u.size for u in other_units], default=0)
        self._n_layer_slots = 3
        self._sym_shards = SymmetricBuffer((total // W) * item, self.group, self.device)
        self._sym_pool = SymmetricBuffer((big + self._n_layer_slots * lay) * item, self.group, self.device)
        self._sym_grad = SymmetricBuffer(total * 4, self.group, self.device)
        self._symm += [self._sym_shards, self._sym_pool, self._sym_grad]
        off = soff = 0
        n_layer = 0
        for u in units:
            shard = u.size // W
            if u.name.startswith("layer"):
                u.slot = 1 + n_layer % self._n_layer_slots
                slot_off = big + (u.slot - 1) * lay
                n_layer += 1
            else:
                u.slot, slot_off = 0, 0
            u.compute = self._sym_pool.view(self.param_dtype, slot_off * item, u.size)
            u.compute_shard = self._sym_shards.view(self.param_dtype, soff * item, shard)
            u.grad = self._sym_grad.view(torch.float32, off * 4, u.size)
            u.grad_ptrs = self._sym_grad.offset_ptr_array(off * 4)
            # the pull kernel copies shard r from ptrs[r] + r * shard_bytes into ptrs[rank] + r * shard_bytes: point
            # every peer entry at its shard buffer minus r shards, and this rank's entry at the slot
            slot_ptr = self._sym_pool.local_ptr + slot_off * item
            u.compute_ptrs = (ctypes.c_void_p * W)(*[
                slot_ptr if r == self.rank else self._sym_shards.peer_ptrs[r] + (soff - r * shard) * item
                for r in range(W)])
            # address that the reduce + AdamW kernel adds shard_lo elements to when it refreshes the bf16 weights
            u.shard_out_ptr = self._sym_shards.local_ptr + (soff - u.shard_lo) * item
            self._alloc_shard_state(u)
            off += u.size
            soff += shard

    def compute_weight_bytes(self) -> int:
        """Bytes of compute-dtype weights this rank keeps allocated (full copy, or shards + slot pool when resharding)."""
        if self.comm != "fused":
            return sum(u.compute.numel() * u.compute.element_size() for u in self.units)
        if self.reshard:
            return self._sym_shards.nbytes + self._sym_pool.nbytes
        return self._sym_compute.nbytes

    def _shards_from_master(self) -> None:
        """Resharded storage: the persistent bf16 shards follow the fp32 master weights; every slot is stale."""
        self.sync_state()
        for u in self.units:
            u.compute_shard.copy_(u.master)
        self._slot_holds, self._resident_ev = {}, {}

    def after_weights_loaded(self) -> None:
        """Called by the loaders after they have written master (and compute) weights."""
        if self.reshard:
            self._shards_from_master()

    # ------------------------------------------------------------------ hooks
    def _install_hooks(self) -> None:
        layers = list(self.model.get_layers_to_shard())
        self._layer_unit = {}
        names = [u.name for u in self.units]
        for i, layer in enumerate(layers):
            ui = names.index(f"layer{i}")
            self._layer_unit[i] = ui
            layer.register_forward_pre_hook(self._make_pre_hook(ui))
        if layers and "head" in names:
            layers[-1].register_forward_hook(self._make_post_hook(names.index("head")))

    def _make_pre_hook(self, ui: int):
        def hook(module, args):
            x, delta = args[0], args[1]
            if self._overlap_active and self._in_backward:
                pass    # recomputation of a checkpointed layer: _backward_residency has made the unit resident
            elif self._overlap_active:
                nxt = ui + 1
                if self.overlap == "gemm2":
                    _lib.flush_pair_gather()              # this unit's weights, if no GEMM of the last layer took them
                    if nxt < len(self.units) and nxt >= 2:
                        self._attach_pair_gather(nxt)
                else:
                    ev = self._gather_done.pop(ui, None)     # this unit's weights were pulled one unit ago
                    if ev is not None:
                        torch.cuda.current_stream(self.device).wait_event(ev)
                    if nxt < len(self.units) and nxt >= 2:
                        self._gather_on_side_stream(nxt)
                if torch.is_grad_enabled() and x.requires_grad:
                    x, delta = _Boundary.apply(self, ui, x, delta)
            return (x, delta) + tuple(args[2:])
        return hook

    def _make_post_hook(self, head_ui: int):
        def hook(module, args, output):
            if self._overlap_active and self.overlap == "gemm2":
                _lib.flush_pair_gather()
            elif self._overlap_active:
                ev = self._gather_done.pop(head_ui, None)
                if ev is not None:
                    torch.cuda.current_stream(self.device).wait_event(ev)
            if self._overlap_active and torch.is_grad_enabled() and output[0].requires_grad:
                return _Boundary.apply(self, ("before", head_ui), output[0], output[1])
            return output
        return hook

    _overlap_active = False

    # ------------------------------------------------------------------ fused communication
    def _unit_flag_index(self, ui: int) -> int:
        return ui * self.world_size

    def _attach_pair_gather(self, ui: int) -> None:
        u = self.units[ui]
        item = u.compute.element_size()
        if getattr(self, "_pair_gather_done", None) is None:     # one scratch array: the launches are stream-ordered
            self._pair_gather_done = torch.zeros(_lib.GATHER_COUNTERS, dtype=torch.int32, device=self.device)
        _lib.attach_pair_gather({
            "peers": u.compute_ptrs, "world": self.world_size, "rank": self.rank,
            "shard_bytes": (u.size // self.world_size) * item,
            "ready": self.pad_weights.local_ptr(self._unit_flag_index(ui)), "epoch": self.epoch, "epoch_add": 0,
            "done": self._pair_gather_done, "base": u.compute.data_ptr(), "nbytes": u.size * item,
            "min_flops": self.pair_gather_min_flops})

    def _gather_on_side_stream(self, ui: int) -> None:
        if self.reshard:     # the slot's previous tenant has been launched on the main stream: start behind it
            ev = torch.cuda.Event()
            ev.record(torch.cuda.current_stream(self.device))
            self.comm_stream.wait_event(ev)
        with torch.cuda.stream(self.comm_stream):
            self._gather_now(ui)
            ev = torch.cuda.Event()
            ev.record(self.comm_stream)
        self._gather_done[ui] = ev

    def _gather_now(self, ui: int) -> None:
        u = self.units[ui]
        if self.reshard:
            if self._slot_holds.get(u.slot) == ui:
                return
            self._slot_holds[u.slot] = ui
            u.compute[u.shard_lo:u.shard_hi].copy_(u.compute_shard)       # own shard: local copy
        _lib.call("ksa_peer_gather", u.compute_ptrs, self.world_size, self.rank, u.size // self.world_size,
                  u.compute.element_size(), self.pad_weights.local_ptr(self._unit_flag_index(ui)), self.epoch, 0, 32)

    def _reduce_args(self, u: Unit, ui: int, state):
        master, exp_avg, exp_avg_sq = state
        return (u.grad_ptrs, self.world_size, self.rank, u.shard_lo, u.shard_hi - u.shard_lo, master, exp_avg,
                exp_avg_sq, self._bf16_out(u), self.hyper, self.beta1,
                self.beta2, self.eps, self.weight_decay, self.clip_value, self.grad_sq,
                self.pad_grads.local_ptr(self._unit_flag_index(ui)), self.epoch, 1)

    def _bf16_out(self, u: Unit):
        if self.param_dtype == torch.float32:
            return None
        return u.shard_out_ptr if self.reshard else u.compute

    def _signal(self, pad, ui: int) -> None:
        pad.set_on_all(self._unit_flag_index(ui) + self.rank, self.epoch, 1)

    def _unit_grads_ready(self, ui: int) -> None:
        """All of this rank's gradients of unit ``ui`` have been launched: tell the peers, then reduce + update."""
        u = self.units[ui]
        for s in u.slots:  # parameters that received no gradient this window contribute zeros
            if not getattr(s.param, "_grad_written", False):
                s.param.main_grad.zero_()
                s.param._grad_written = True
        main = torch.cuda.current_stream(self.device)
        ev = torch.cuda.Event()
        ev.record(main)
        with torch.cuda.stream(self.comm_stream):
            self.comm_stream.wait_event(ev)
            self._signal(self.pad_grads, ui)
            with self._optimizer_state(u) as state:
                # one CTA per SM: fits beside a GEMM CTA
                _lib.call("ksa_peer_reduce_adamw", *self._reduce_args(u, ui, state), 148)
            self._signal(self.pad_weights, ui)
        self._done_units.add(ui)

    def _backward_residency(self, tag) -> None:
        """Resharded storage: the backward pass of the unit in front of ``tag`` runs next; make its weights resident
        (a later unit may have taken its slot) and start pulling the one before it."""
        if not (self.reshard and self._overlap_active):
            return
        self._in_backward = True
        nxt = (tag[1] if isinstance(tag, tuple) else tag) - 1      # unit whose backward pass starts now
        main = torch.cuda.current_stream(self.device)
        for ui in (nxt, nxt - 1):
            if ui < 1 or not self.units[ui].name.startswith("layer"):
                continue                                            # the embedding's backward pass reads no weights
            if self._slot_holds.get(self.units[ui].slot) != ui:
                ev = torch.cuda.Event()
                ev.record(main)                                     # whoever used the slot before has been launched
                with torch.cuda.stream(self.comm_stream):
                    self.comm_stream.wait_event(ev)
                    self._gather_now(ui)
                    done = torch.cuda.Event()
                    done.record(self.comm_stream)
                self._resident_ev[ui] = done
        ev = self._resident_ev.pop(nxt, None)
        if ev is not None:
            main.wait_event(ev)

    def _backward_reached(self, tag) -> None:
        if not self._is_boundary_step:
            return
        if isinstance(tag, tuple):          # ("before", head): the head's gradients are complete
            self._unit_grads_ready(tag[1])
            return
        self._unit_grads_ready(tag)         # backward of layer unit `tag` has been launched

    # ------------------------------------------------------------------ step
    def _write_hyper(self) -> None:
        super()._write_hyper()
        slot = (self._hyper_slot - 1) % len(self._hyper_events)   # same slot and event as the hyper-parameters
        self._epoch_ring[slot, 0] = self._flag_epoch
        self.epoch.copy_(self._epoch_ring[slot], non_blocking=True)
        if self.device.type == "cuda":
            ev = torch.cuda.Event()
            ev.record(torch.cuda.current_stream(self.device))
            self._hyper_events[slot] = ev

    def forward_backward(self, tokens, labels, **kw):
        if self.comm != "fused":
            return super().forward_backward(tokens, labels, **kw)
        self._is_boundary_step = self.micro_step + 1 == self.grad_accum_steps
        if self.micro_step == 0:
            self.grad_sq.zero_()
        self._done_units = set()
        self._overlap_active = True
        self._in_backward = False
        try:
            if self.micro_step == 0:          # refreshed weights of the first two units; later ones are pulled ahead
                main = torch.cuda.current_stream(self.device)
                if not torch.cuda.is_current_stream_capturing():
                    # the previous step's updates of this rank's own shards; inside a graph the previous replay has
                    # joined the side stream already, and a stream outside the capture cannot be waited on
                    main.wait_stream(self.comm_stream)
                self.comm_stream.wait_stream(main)
                self._gather_now(0)
                if len(self.units) > 1:
                    self._gather_now(1)
            return super().forward_backward(tokens, labels, **kw)
        finally:
            self._overlap_active = False

    def train_step(self, tokens, labels, **kw):
        self._write_hyper()   # the optimizer runs inside backward and gathers read the epoch: both must be there first
        if self.micro_step == 0:
            self.zero_grad()
        if tokens.device != self.device:
            tokens = tokens.to(self.device, non_blocking=True)
            labels = labels.to(self.device, non_blocking=True)
        if self.micro_step == 0:
            self.grad_sq.zero_()
        loss = self.forward_backward(tokens, labels, **kw)
        self.micro_step += 1
        if self.micro_step == self.grad_accum_steps:
            self.optimizer_step()
            self.step_count += 1
            self.micro_step = 0
        return loss

    def optimizer_step(self) -> None:
        self._grad_sq_reduced = None
        if self.comm == "fused":
            self._collect_autograd_grads()
            for ui in range(len(self.units) - 1, -1, -1):   # whatever backward did not reach (embed; all, if hooks are off)
                if ui not in self._done_units:
                    self._unit_grads_ready(ui)
            torch.cuda.current_stream(self.device).wait_stream(self.comm_stream)
            self._flag_epoch += 1
            self._slot_holds, self._resident_ev = {}, {}      # resharded storage: every slot holds old weights now
            return
        self._collect_autograd_grads()
        self.grad_sq.zero_()
        for unit in reversed(self.units):
            self._reduce_and_update(unit)

    def _reduce_and_update(self, unit: Unit) -> None:
        """Collective path: reduce-scatter -> AdamW on the shard -> all-gather of the refreshed weights."""
        w = self.world_size
        lo, hi = unit.shard_lo, unit.shard_hi
        if w > 1:
            backend = dist.get_backend(self.group)
            if backend == "nccl":
                shard = torch.empty(hi - lo, dtype=torch.float32, device=self.device)
                dist.reduce_scatter_tensor(shard, unit.grad, group=self.group)
            else:
                dist.all_reduce(unit.grad, group=self.group)
                shard = unit.grad[lo:hi]
        else:
            shard = unit.grad[lo:hi]
        out = unit.compute[lo:hi] if self.param_dtype != torch.float32 else None
        with self._optimizer_state(unit) as (master, exp_avg, exp_avg_sq):
            ops.adamw_step(master, shard, exp_avg, exp_avg_sq, out, self.hyper, self.beta1, self.beta2,
                           self.eps, self.weight_decay, self.clip_value, self.grad_sq)
            if self.param_dtype == torch.float32:
                unit.compute[lo:hi].copy_(master)
        if w > 1:
            if dist.get_backend(self.group) == "nccl":
                dist.all_gather_into_tensor(unit.compute, unit.compute[lo:hi].clone(), group=self.group)
            else:
                parts = [torch.empty(hi - lo, dtype=unit.compute.dtype, device=self.device) for _ in range(w)]
                dist.all_gather(parts, unit.compute[lo:hi].contiguous(), group=self.group)
                unit.compute.copy_(torch.cat(parts))

    def grad_norm(self) -> torch.Tensor:
        """Global gradient norm: shard-local sums of squares, one scalar all-reduce (``muse/training/common.py:273-326``)."""
        if self._grad_sq_reduced is None:
            t = self.grad_sq.clone()
            if self.world_size > 1:
                dist.all_reduce(t, group=self.group)
            self._grad_sq_reduced = t
        return self._grad_sq_reduced.sqrt()

    def graphed_step(self, tokens, labels):
        """Only the collective back end can be replayed from a CUDA graph.  The fused step is not captured: its
        communication kernels wait on flags raised by other GPUs and sit on a side-stream branch; a graph replay is
        free to order independent branches as it likes, and with four ranks it ordered a waiting kernel ahead of the
        kernel its peers were waiting for (a distributed deadlock that only the bounded waits ended).  The eager step
        with explicit streams keeps the launch order that the protocol assumes."""
        if self.comm == "fused":
            return self.train_step(tokens, labels)
        return super().graphed_step(tokens, labels)

    def refresh_compute_from_master(self) -> None:
        if self.reshard:
            return self._shards_from_master()
        self.sync_state()
        for u in self.units:
            u.compute[u.shard_lo:u.shard_hi].copy_(u.master)
            if self.world_size > 1:
                parts = [torch.empty(u.shard_hi - u.shard_lo, dtype=u.compute.dtype, device=self.device)
                         for _ in range(self.world_size)]
                dist.all_gather(parts, u.compute[u.shard_lo:u.shard_hi].contiguous(), group=self.group)
                u.compute.copy_(torch.cat(parts))

    def close(self) -> None:
        if self.comm == "fused":
            _lib.take_pair_gather()     # a gather still waiting for a GEMM would name buffers that are freed below
            torch.cuda.synchronize(self.device)
            self.pad_grads.close()
            self.pad_weights.close()
            for s in self._symm:
                s.close()
            self._symm = []
