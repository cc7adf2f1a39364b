"""Tensor parallelism for inference (TP 1/2/4/8; the reference serves its models through vLLM's tensor-parallel
workers, ``examples/inference/README.md``; this package carries its own engine).

Each rank holds ``Hq/T`` query heads, ``Hkv/T`` key/value heads (and their KV caches), ``F/T`` feed-forward columns and
``V/T`` rows of the output head; the residual stream is replicated.  The QKV and gate/up projections are
column-parallel (no communication).  The attention output and the down projection are row-parallel: every rank's
GEMM writes its partial ``[rows, D]`` block straight into a symmetric-memory slot, and ONE kernel
(``ksa_tp_allreduce_add_rmsnorm``) announces the block, waits (bounded) for the peers', sums all partials row by row
over P2P loads in rank order, adds the residual row and applies the next RMSNorm: the all-reduce never exists as a
separate pass and every rank keeps a bit-identical residual stream.

CPU (gloo) ranks run the same layout with ``all_reduce`` / ``all_gather`` for the tests.
"""
from __future__ import annotations

import ctypes
import os
from typing import Dict, Optional, Tuple

import torch
import torch.distributed as dist

from .. import ops
from ..ops import _lib


class TpContext:
    """Group + (on GPUs) the symmetric partial-sum slots of one tensor-parallel group."""

    def __init__(self, group, embed_dim: int, max_rows: int, device=None, dtype=torch.bfloat16,
                 two_phase_rows: int = 2048, two_phase_min_size: Optional[int] = None,
                 fused_gather: Optional[bool] = None, push_partials: Optional[bool] = None):
        if two_phase_min_size is None:
            two_phase_min_size = int(os.environ.get("KSA_TP_TWO_PHASE_MIN", "3"))
        self.group = group
        self.rank = dist.get_rank(group)
        self.size = dist.get_world_size(group)
        if fused_gather is None:
            # measured: the launch that gathers inside the GEMM is 1.7-1.8 x faster than gather kernel + GEMM on its
            # own (2 and 4 GPUs), but a whole 32768-token prefill of KSA-4B on 4 GPUs takes 139.5 ms with it against
            # 134.4-137.9 ms without (three runs each on one box), so groups of more than two gather separately
            env = os.environ.get("KSA_TP_FUSED_GATHER")
            fused_gather = (env == "1") if env is not None else self.size <= 2
        if push_partials is None:
            # measured (33024 x 2560 x 2048, GEMM + reduction): scattering from the epilogue wins on 2 GPUs (0.40 against
            # 0.45 ms) and loses on 4 (0.50 against 0.47 ms), where the blocks of one tile go to four owners
            env = os.environ.get("KSA_TP_PUSH_PARTIALS")
            push_partials = (env == "1") if env is not None else self.size <= 2
        self.D = embed_dim
        self.max_rows = max_rows
        self.device = device
        self.dtype = dtype
        self.fused = self._on_gpus(device)
        self.counter = 0            # all-reduces issued so far (identical on every rank)
        self.two_phase_rows = 0
        self.fused_gather = False
        self._pending = None          # (data_ptr of the normalised rows, shard rows, rows) awaiting their gather
        self._res_event = None        # end of the residual gather on the side stream
        self.push_partials = False
        self._pushed = None           # (slot, shard rows, residual rows) of a row-parallel GEMM that scattered its rows
        if self.fused:
            from .symm import SignalPad, SymmetricBuffer
            item = torch.empty((), dtype=dtype).element_size()
            # + size rows: the scattered layout of a slot holds size blocks of ceil(rows / size) rows
            self.slot_bytes = ((max_rows + self.size) * embed_dim * item + 255) // 256 * 256
            self.buf = SymmetricBuffer(2 * self.slot_bytes, group, device)
            self.flags = SignalPad(self.size, group, device)
            self.flags.flags.zero_()
            torch.cuda.synchronize(device)
            dist.barrier(group)
            self._slot_ptrs = [self.buf.offset_ptr_array(s * self.slot_bytes) for s in range(2)]
            self._announce = self.flags.flag_ptrs(self.rank)
            # [finished all-reduces, finished CTAs of the running one]: on the device, so that a captured CUDA graph
            # of a decode step stays valid while the exchange number advances
            self._epoch = torch.zeros(2, dtype=torch.int32, device=device)
            # Two-phase all-reduce for many rows (prefill) on groups of 3 or more: reduce-scatter + add + norm of this
            # rank's row shard into symmetric residual / normalised buffers, then a P2P gather of the peers' shards.
            # Each rank then reads 3 x rows x D elements instead of T x rows x D.
            self.two_phase_rows = (two_phase_rows if self.size >= two_phase_min_size and two_phase_rows > 0
                                   and max_rows >= two_phase_rows else 0)
            if self.two_phase_rows:
                self.rows_pad = (max_rows + self.size - 1) // self.size * self.size
                plane = (self.rows_pad * embed_dim * item + 255) // 256 * 256
                self._plane_bytes = plane
                self.sp_buf = SymmetricBuffer(2 * plane, group, device)          # [residual | normalised]
                self.flags2 = SignalPad(self.size, group, device)
                self._notify = self.flags2.flag_ptrs(self.rank)
                self._res_ptrs = self.sp_buf.offset_ptr_array(0)
                self._y_ptrs = self.sp_buf.offset_ptr_array(plane)
            # All-gather -> GEMM in one launch for the normalised rows (the column-parallel projection that follows
            # reads them shard by shard as they land); the residual rows travel on a side stream meanwhile.
            self.fused_gather = bool(fused_gather) and bool(self.two_phase_rows)
            # GEMM -> reduce-scatter: the row-parallel GEMM's epilogue stores every row block into its owner's slot
            self.push_partials = bool(push_partials) and bool(self.two_phase_rows)
            if self.fused_gather:
                self._done = torch.zeros(_lib.GATHER_COUNTERS, dtype=torch.int32, device=device)
                self._side = torch.cuda.Stream(device=device)

    @staticmethod
    def _on_gpus(device) -> bool:
        """Whether the group exchanges through symmetric memory and the fused kernels (else: collectives)."""
        return device is not None and torch.device(device).type == "cuda"

    def close(self) -> None:
        if self.fused:
            self.flush()
            torch.cuda.synchronize(self.device)
            dist.barrier(self.group)
            self.flags.close()
            self.buf.close()
            if self.two_phase_rows:
                self.flags2.close()
                self.sp_buf.close()

    # ------------------------------------------------------------------ row-parallel linear + fused all-reduce
    def _slot_view(self, rows: int) -> torch.Tensor:
        if rows > self.max_rows:
            raise ValueError(f"{rows} rows exceed the tensor-parallel exchange buffer ({self.max_rows} rows)")
        return self.buf.view(self.dtype, (self.counter % 2) * self.slot_bytes, rows * self.D).view(rows, self.D)

    def row_parallel_linear(self, x: torch.Tensor, weight: torch.Tensor,
                            residual_rows: Optional[int] = None) -> torch.Tensor:
        """Partial ``x_local @ weight_local.T``; on GPUs written into the slot the next all-reduce reads.

        ``residual_rows``: rows of the residual stream that the following ``add_rms_norm`` will get.  With it the
        two-phase form is known in advance and the GEMM can scatter its row blocks into the owners' slots
        (``ksa_gemm2_scatter_bf16``); the returned tensor is then only a token for ``add_rms_norm``."""
        if not self.fused:
            return ops.linear(x, weight)
        self.flush()
        out = self._slot_view(x.shape[0])
        x = x if x.is_contiguous() else x.contiguous()
        if (self.push_partials and residual_rows is not None and residual_rows >= self.two_phase_rows
                and residual_rows >= x.shape[0] and weight.stride(1) == 1):
            T, D, item = self.size, self.D, x.element_size()
            s = self.counter % 2
            shard = (residual_rows + T - 1) // T
            # rank r's slot s holds T blocks of `shard` rows: block q is rank q's partial of r's rows
            targets = (ctypes.c_void_p * T)(*[p + s * self.slot_bytes + self.rank * shard * D * item
                                              for p in self.buf.peer_ptrs])
            _lib.call("ksa_gemm2_scatter_bf16", x, weight, x.shape[0], weight.shape[0], x.shape[1], x.stride(0),
                      weight.stride(0), D, targets, T, shard)
            self._pushed = (s, shard, residual_rows)
            return out
        self._pushed = None
        ops.gemm(x, weight, out=out)
        return out

    def add_rms_norm(self, x: torch.Tensor, partial: torch.Tensor, weight: torch.Tensor,
                     eps: float, defer_gather: bool = False) -> Tuple[torch.Tensor, torch.Tensor]:
        """``r = x + sum_ranks(partial)`` on the first ``partial.shape[0]`` rows and ``rms_norm(r)``.

        ``defer_gather``: the caller promises that the next reader of the normalised rows is
        ``col_parallel_linear`` and that it reads the residual rows only after another call into this object (or
        ``flush``); the gathers of the two-phase form may then overlap with what follows."""
        if not self.fused:
            total = partial.clone()
            dist.all_reduce(total, group=self.group)
            return ops.add_rms_norm(x, total, weight, eps)
        self.flush()
        rows_x, rows_d = x.shape[0], partial.shape[0]
        slot = self._slot_view(rows_d)
        pushed, self._pushed = self._pushed, None
        if partial.data_ptr() != slot.data_ptr():
            pushed = None
            slot.copy_(partial)
        x = x if x.is_contiguous() else x.contiguous()
        s = self.counter % 2
        self.counter += 1
        if pushed is not None and (pushed[0] != s or pushed[2] != rows_x):
            raise RuntimeError(f"the row-parallel GEMM scattered its rows for a residual of {pushed[2]} rows, "
                               f"but add_rms_norm got {rows_x}")
        if self.two_phase_rows and rows_x >= self.two_phase_rows:
            return self._two_phase(x, s, weight, rows_x, rows_d, eps, defer_gather and self.fused_gather,
                                   pushed is not None)
        res = torch.empty_like(x)
        y = torch.empty_like(x)
        _lib.call("ksa_tp_allreduce_add_rmsnorm", x, self._slot_ptrs[s], self._announce, self.flags.local_ptr(0),
                  self.size, self.rank, weight, res, y, rows_x, rows_d, self.D, float(eps), self._epoch[0:1],
                  self._epoch[1:2])
        return res, y

    def _two_phase(self, x, s, weight, rows_x, rows_d, eps, defer=False, pushed=False):
        """Reduce-scatter + add + norm of this rank's rows, then gather of the peers' rows.  The results live in the
        symmetric buffers until the next call of this kind (the callers consume them before that)."""
        T, D = self.size, self.D
        shard = (rows_x + T - 1) // T
        lo, hi = min(self.rank * shard, rows_x), min((self.rank + 1) * shard, rows_x)
        res = self.sp_buf.view(self.dtype, 0, self.rows_pad * D).view(self.rows_pad, D)
        y = self.sp_buf.view(self.dtype, self._plane_bytes, self.rows_pad * D).view(self.rows_pad, D)
        partials = self._slot_ptrs[s]
        if pushed:
            # every rank's partial of MY rows already sits in my own slot (block q from rank q): local reads only.
            # The kernel indexes by global row, hence the bias by the first own row.
            item = x.element_size()
            base = self.buf.local_ptr + s * self.slot_bytes - lo * D * item
            partials = (ctypes.c_void_p * T)(*[base + q * shard * D * item for q in range(T)])
        _lib.call("ksa_tp_reduce_scatter_add_rmsnorm", x, partials, self._announce, self.flags.local_ptr(0),
                  T, self.rank, weight, res, y, rows_x, rows_d, D, float(eps), self._epoch[0:1], self._epoch[1:2],
                  lo, hi, self._notify)
        # the epoch was advanced by the kernel above (stream order): a peer's shard is complete once its flag reached it
        if defer:
            main = torch.cuda.current_stream()
            self._side.wait_stream(main)
            with torch.cuda.stream(self._side):
                _lib.call("ksa_peer_gather", self._res_ptrs, T, self.rank, shard * D, x.element_size(),
                          self.flags2.local_ptr(0), self._epoch[0:1], 0, 16)
                self._res_event = torch.cuda.Event()
                self._res_event.record(self._side)
            self._pending = (y.data_ptr(), shard, rows_x)
            return res[:rows_x], y[:rows_x]
        for ptrs in (self._res_ptrs, self._y_ptrs):
            _lib.call("ksa_peer_gather", ptrs, T, self.rank, shard * D, x.element_size(), self.flags2.local_ptr(0),
                      self._epoch[0:1], 0, 32)
        return res[:rows_x], y[:rows_x]

    # ------------------------------------------------------------------ deferred gathers of the two-phase form
    def flush(self) -> None:
        """Complete what ``add_rms_norm(..., defer_gather=True)`` left open: gather the normalised rows now if no
        projection took them along, and make the current stream wait for the residual rows."""
        if not self.fused_gather:
            return
        if self._pending is not None:
            _, shard, _ = self._pending
            self._pending = None
            _lib.call("ksa_peer_gather", self._y_ptrs, self.size, self.rank, shard * self.D,
                      torch.empty((), dtype=self.dtype).element_size(), self.flags2.local_ptr(0), self._epoch[0:1], 0, 32)
        if self._res_event is not None:
            torch.cuda.current_stream().wait_event(self._res_event)
            self._res_event = None

    def col_parallel_linear(self, h: torch.Tensor, weight: torch.Tensor,
                            out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """``h @ weight_local.T``.  When ``h`` is the normalised output of a deferred two-phase ``add_rms_norm``, the
        gather of the other ranks' rows of ``h`` runs inside the GEMM launch (``ksa_gemm2_gather_bf16``)."""
        p = self._pending if self.fused_gather else None
        if (p is None or h.data_ptr() != p[0] or h.dim() != 2 or not h.is_contiguous() or h.shape[0] > p[2]
                or h.shape[1] != self.D or weight.stride(1) != 1
                or (torch.is_grad_enabled() and (h.requires_grad or weight.requires_grad))):
            self.flush()
            if out is not None:
                return ops.gemm(h, weight, out=out)
            return ops.linear(h, weight)
        _, shard, _ = p
        self._pending = None
        return ops.gemm_gather(h, weight, self._y_ptrs, self.size, self.rank, shard * self.D * h.element_size(),
                               self.flags2.local_ptr(0), self._epoch[0:1], self._done, dep_operand=1, dep_offset=0,
                               out=out)

    # ------------------------------------------------------------------ vocabulary-parallel head
    def gather_logits(self, local: torch.Tensor) -> torch.Tensor:
        """``[..., V/T]`` per rank -> ``[..., V]`` (rank order)."""
        self.flush()
        parts = [torch.empty_like(local) for _ in range(self.size)]
        dist.all_gather(parts, local.contiguous(), group=self.group)
        return torch.cat(parts, dim=-1)


# ---------------------------------------------------------------------- sharding
def tp_local_config(cfg, size: int):
    """The per-rank model configuration: heads and feed-forward columns divided by the group size."""
    if cfg.num_heads % size or cfg.num_kv_heads % size or cfg.intermediate_dim % size:
        raise ValueError(f"heads {cfg.num_heads}/{cfg.num_kv_heads} and FFN {cfg.intermediate_dim} must divide by TP {size}")
    return cfg.merge({"num_heads": cfg.num_heads // size, "num_kv_heads": cfg.num_kv_heads // size,
                      "intermediate_dim": cfg.intermediate_dim // size})


def shard_state_dict(state: Dict[str, torch.Tensor], cfg, rank: int, size: int,
                     shard_head: bool = True) -> Dict[str, torch.Tensor]:
    """Slice a whole-model state dict (this package's fused parameter names) for one rank."""
    Hq, Hkv, Dh, F = cfg.num_heads, cfg.num_kv_heads, cfg.head_dim, cfg.intermediate_dim
    hq, hkv, f = Hq // size, Hkv // size, F // size
    out: Dict[str, torch.Tensor] = {}
    for k, v in state.items():
        if k.endswith("attn.wqkv.weight") or k.endswith("attn.wqkv_summary.weight"):
            q, kk, vv = v[:Hq * Dh], v[Hq * Dh:(Hq + Hkv) * Dh], v[(Hq + Hkv) * Dh:]
            out[k] = torch.cat([q[rank * hq * Dh:(rank + 1) * hq * Dh], kk[rank * hkv * Dh:(rank + 1) * hkv * Dh],
                                vv[rank * hkv * Dh:(rank + 1) * hkv * Dh]], dim=0).contiguous()
        elif k.endswith("attn.output_proj.weight"):
            out[k] = v[:, rank * hq * Dh:(rank + 1) * hq * Dh].contiguous()
        elif k.endswith("mlp.w13.weight"):
            out[k] = torch.cat([v[rank * f:(rank + 1) * f], v[F + rank * f:F + (rank + 1) * f]], dim=0).contiguous()
        elif k.endswith("mlp.w2.weight"):
            out[k] = v[:, rank * f:(rank + 1) * f].contiguous()
        elif k == "output.weight" and shard_head and v.shape[0] % size == 0:
            n = v.shape[0] // size
            out[k] = v[rank * n:(rank + 1) * n].contiguous()
        else:
            out[k] = v
    return out


def build_tp_model(full_state: Dict[str, torch.Tensor], cfg, tp: TpContext, device=None, dtype=None):
    """Instantiate this rank's shard of a model from a whole-model state dict and attach ``tp`` to it."""
    from ..models import get_model_class
    local_cfg = tp_local_config(cfg, tp.size)
    with torch.device("meta"):
        model = get_model_class(cfg.model_class)(local_cfg)
    shard = shard_state_dict(full_state, cfg, tp.rank, tp.size)
    if "output.weight" in shard and model.output is not None and shard["output.weight"].shape[0] != cfg.vocab_size:
        model.output.weight = torch.nn.Parameter(torch.empty(shard["output.weight"].shape, device="meta"))
    model = model.to_empty(device=device or "cpu")
    model.load_state_dict(shard, strict=True)
    if dtype is not None:
        model = model.to(dtype)
    model.tp = tp
    return model
