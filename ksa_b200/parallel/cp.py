"""Context parallelism by locality for Kwai Summary Attention.

The reference shards the sequence with DeepSpeed-Ulysses: four all-to-alls per attention layer move every q, k, v and
output row between ranks (``muse/training/parallel.py:211-335``, ``muse/models/qwen3_sa/_layers.py:179-224``).  KSA
needs far less: rank ``r`` of a group of ``P`` owns the contiguous, chunk-aligned text rows
``[r*Ll, (r+1)*Ll)`` and the summary rows of those chunks, and for a summary-attention layer with a window of ``W``
chunks its queries only see

* the last ``W*C`` text keys before its shard (a halo owned by rank ``r-1``, and further back only when the window
  is longer than a shard), and
* the summary keys of every earlier chunk (``S`` rows per chunk: tiny).

So each rank stages ``[halo | own text]`` and ``[older summaries | own summaries]`` K/V buffers and runs the same
attention kernels with index offsets (``q_off / k_off / s_off``).  In backward the gradients that land on halo and
older-summary rows are returned to their owners, who add them.  Full-attention layers of a hybrid stack stage all
earlier text K/V (the halo is everything before the shard).

Transport:
* GPUs, summary layers (the default when the shapes are tile-aligned, ``_CpDirectAttention``): every rank copies its
  K/V rows into its symmetric exchange slot and raises a flag; the attention kernels then read the halo tiles and
  the older summaries' tiles STRAIGHT FROM THE OWNERS' SLOTS with their own TMA loads (``ksa_attn_fwd_cp``,
  ``ksa_attn_bwd_fused_cp``: peer tiles stream in while the local block pairs are computed), and the backward
  kernel adds the dK / dV of keys it does not own into the owners' fp32 return blocks over NVLink from its epilogue;
  the owner folds its return block into its gradients (a local pass).  No staging copies, no NCCL collective.
* GPUs, other cases (windows longer than a shard, summary counts that do not fill key tiles, the bit-reproducible
  mode, full-attention layers in ``halo`` mode): consumers pull the ranges they need into staging buffers with P2P
  copy kernels (``ksa_peer_copy`` / ``ksa_peer_add_bf16``), ordered by per-rank flags; each wait is bounded.
* CPU (gloo) ranks, used by the tests: the same staging expressed with ``all_gather`` / ``all_reduce``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Tuple

import torch
import torch.distributed as dist

from .. import ops
from ..ops import _lib, reference as ref
from ..ops.layout import two_stream_masks


@dataclass
class CpShape:
    """Static description of one rank's shard."""
    rank: int
    size: int
    seq_len: int      # global text length L
    chunk: int
    n_sum: int

    @property
    def local_len(self) -> int:
        return self.seq_len // self.size

    @property
    def local_chunks(self) -> int:
        return self.local_len // self.chunk

    @property
    def local_sum(self) -> int:
        return self.local_chunks * self.n_sum

    def check(self) -> None:
        if self.seq_len % self.size or self.local_len % self.chunk:
            raise ValueError(f"sequence {self.seq_len} must split into {self.size} chunk-aligned shards (chunk {self.chunk})")

    def halo_len(self, window_chunks: Optional[int]) -> int:
        """Text keys before the shard that its queries can see (``None`` = full attention: everything)."""
        before = self.rank * self.local_len
        if window_chunks is None:
            return before
        return min(before, window_chunks * self.chunk)


class CpContext:
    """Group, shard shape and (on GPUs) the symmetric exchange buffers of one context-parallel group."""

    def __init__(self, group, seq_len: int, chunk: int, n_sum: int, n_kv_heads: int, head_dim: int, batch: int = 1,
                 device=None, dtype=torch.bfloat16, full_layers: bool = False, max_window: int = 8,
                 n_heads: Optional[int] = None, full_layer_mode: str = "auto"):
        self.group = group
        self.rank = dist.get_rank(group)
        self.size = dist.get_world_size(group)
        self.shape = CpShape(self.rank, self.size, seq_len, chunk, n_sum)
        self.shape.check()
        self.batch = batch
        self.kv_width = 2 * n_kv_heads * head_dim          # K | V per row
        self.device = device
        self.fused = self._on_gpus(device)
        self.counter = 0                                    # forward exchanges issued so far (same on every rank)
        self.counter_bwd = 0                                # backward exchanges (they use their own slots and flags)
        self.slot_last = [None, None, None, None]           # exchange number of each slot's previous use
        # full-attention layers: "ulysses" reshards sequence -> heads around the attention (balanced causal work),
        # "halo" stages every earlier key in front of the shard (rank r does (2r+1)/P^2 of the work)
        self.n_heads, self.n_kv_heads, self.head_dim = n_heads, n_kv_heads, head_dim
        can_ulysses = n_heads is not None and n_heads % self.size == 0 and n_kv_heads % self.size == 0
        if full_layer_mode == "auto":
            full_layer_mode = "ulysses" if can_ulysses else "halo"
        if full_layer_mode == "ulysses" and not can_ulysses:
            raise ValueError(f"head-parallel full-attention layers need heads ({n_heads}/{n_kv_heads}) divisible by {self.size}")
        self.full_layer_mode = full_layer_mode
        self.a2a_counter = 0
        self.a2a_slot_last = [None, None]
        if full_layer_mode == "ulysses":
            full_layers = False                             # no gradient return blocks of whole shards are needed
        if self.fused:
            from .symm import SignalPad, SymmetricBuffer
            rows = batch * (self.shape.local_len + self.shape.local_sum)
            item = torch.empty((), dtype=dtype).element_size()
            self.rows = rows
            self.slot_bytes = rows * self.kv_width * item
            # two slots for forward K/V blocks, two (sized for the largest halo) for returned gradients
            self.ret_slot_bytes = max(_ret_rows(self.shape, batch, full_layers, max_window), 1) * self.kv_width * item
            self.xbuf = SymmetricBuffer(2 * self.slot_bytes + 2 * self.ret_slot_bytes, group, device)
            self.ready = SignalPad(4 * self.size, group, device)      # [slot][producer rank] <- exchange number + 1
            self.consumed = SignalPad(4 * self.size, group, device)   # [slot][consumer rank] <- exchange number + 1
            self.dtype = dtype
            # direct mode: [2 forward K/V slots | 2 backward K/V slots | 2 fp32 return blocks], flags per (slot, rank)
            self.d_fwd = self.d_bwd = 0
            self.d_slot_last = [None] * 6
            self.d_halo_max = min(max_window * chunk, self.shape.local_len)
            self.d_ret_bytes = batch * (self.d_halo_max + self.shape.local_sum) * self.kv_width * 4
            self.dbuf = SymmetricBuffer(4 * self.slot_bytes + 2 * self.d_ret_bytes, group, device)
            self.dready = SignalPad(6 * self.size, group, device)
            self.dconsumed = SignalPad(6 * self.size, group, device)
            self.a2a_buf = None
            if self.full_layer_mode == "ulysses":
                width = (n_heads + 2 * n_kv_heads) * head_dim
                self.a2a_slot_bytes = batch * self.shape.local_len * width * item
                self.a2a_buf = SymmetricBuffer(2 * self.a2a_slot_bytes, group, device)
                self.a2a_ready = SignalPad(2 * self.size, group, device)
                self.a2a_consumed = SignalPad(2 * self.size, group, device)

    @staticmethod
    def _on_gpus(device) -> bool:
        """Whether the group exchanges through symmetric memory and P2P kernels (else: collectives)."""
        return device is not None and torch.device(device).type == "cuda"

    def close(self) -> None:
        if self.fused:
            torch.cuda.synchronize(self.device)
            self.ready.close()
            self.consumed.close()
            self.xbuf.close()
            self.dready.close()
            self.dconsumed.close()
            self.dbuf.close()
            if self.a2a_buf is not None:
                self.a2a_ready.close()
                self.a2a_consumed.close()
                self.a2a_buf.close()

    # ------------------------------------------------------------------ ranges
    def text_sources(self, halo: int) -> List[Tuple[int, int, int]]:
        """Halo rows as ``(owner rank, first local row, n rows)`` in global order."""
        Ll = self.shape.local_len
        out = []
        start = self.rank * Ll - halo
        while halo > 0:
            owner = start // Ll
            lo = start - owner * Ll
            n = min(Ll - lo, halo)
            out.append((owner, lo, n))
            start += n
            halo -= n
        return out


def _ret_rows(shape: CpShape, batch: int, full_layers: bool, max_window: int) -> int:
    halo = (shape.size - 1) * shape.local_len if full_layers else min((shape.size - 1) * shape.local_len,
                                                                      max_window * shape.chunk)
    return batch * (halo + (shape.size - 1) * shape.local_sum)


class _CpStage(torch.autograd.Function):
    """``kv_local`` ``[B*Ll + B*Nsl, 2*Hkv*D]`` -> (``[B, halo+Ll, kvw]`` text K|V, ``[B, (r+1)*Nsl, kvw]`` summary K|V).

    Backward returns the gradients of halo / older-summary rows to their owners and adds what later ranks return.
    """

    @staticmethod
    def forward(ctx, kv_local, cp: CpContext, window_chunks: Optional[int], summaries: bool):
        sh, B = cp.shape, cp.batch
        Ll, Nsl, r, P, kvw = sh.local_len, sh.local_sum, cp.rank, cp.size, cp.kv_width
        halo = sh.halo_len(window_chunks)
        ctx.cp, ctx.halo, ctx.summaries = cp, halo, summaries
        ctx.halo_of = lambda q: CpShape(q, sh.size, sh.seq_len, sh.chunk, sh.n_sum).halo_len(window_chunks)
        if not summaries:
            Nsl = 0
        text_local = kv_local[:B * Ll].view(B, Ll, kvw)
        sum_local = kv_local[B * Ll:].view(B, Nsl, kvw)
        st_text = kv_local.new_empty(B, halo + Ll, kvw)
        st_sum = kv_local.new_empty(B, (r + 1) * Nsl, kvw)
        st_text[:, halo:] = text_local
        st_sum[:, r * Nsl:] = sum_local
        if not cp.fused:
            parts = [torch.empty_like(kv_local) for _ in range(P)]
            dist.all_gather(parts, kv_local.contiguous(), group=cp.group)
            for owner, lo, n in cp.text_sources(halo):
                off = (owner * Ll + lo) - (r * Ll - halo)
                st_text[:, off:off + n] = parts[owner][:B * Ll].view(B, Ll, kvw)[:, lo:lo + n]
            for p in range(r):
                st_sum[:, p * Nsl:(p + 1) * Nsl] = parts[p][B * Ll:].view(B, Nsl, kvw)
            return st_text, st_sum
        e = cp.counter
        cp.counter += 1
        slot = e % 2
        item = kv_local.element_size()
        row_b = kvw * item
        if cp.slot_last[slot] is not None:   # every consumer has finished reading this slot's previous contents
            cp.consumed.wait_local(slot * P, P, None, cp.slot_last[slot] + 1)
        cp.slot_last[slot] = e
        cp.xbuf.view(cp.dtype, slot * cp.slot_bytes, kv_local.numel()).copy_(kv_local.reshape(-1))
        cp.ready.set_on_all(slot * P + r, None, e + 1)
        base = slot * cp.slot_bytes
        for owner, lo, n in cp.text_sources(halo):
            off = (owner * Ll + lo) - (r * Ll - halo)
            for b in range(B):
                _lib.call("ksa_peer_copy", st_text[b, off:off + n], cp.xbuf.peer_ptrs[owner] + base + (b * Ll + lo) * row_b,
                          n * row_b, cp.ready.local_ptr(slot * P + owner), None, e + 1, 16)
        if Nsl > 0:
            for p in range(r):
                for b in range(B):
                    _lib.call("ksa_peer_copy", st_sum[b, p * Nsl:(p + 1) * Nsl],
                              cp.xbuf.peer_ptrs[p] + base + (B * Ll + b * Nsl) * row_b, Nsl * row_b,
                              cp.ready.local_ptr(slot * P + p), None, e + 1, 8)
        cp.consumed.set_on_all(slot * P + r, None, e + 1)
        return st_text, st_sum

    @staticmethod
    def backward(ctx, g_text, g_sum):
        cp, halo = ctx.cp, ctx.halo
        sh, B = cp.shape, cp.batch
        Ll, Nsl, r, P, kvw = sh.local_len, sh.local_sum, cp.rank, cp.size, cp.kv_width
        if not ctx.summaries:
            Nsl = 0
        g_text = g_text.contiguous()
        g_sum = g_sum.contiguous()
        g_local = torch.cat([g_text[:, halo:].reshape(B * Ll, kvw), g_sum[:, r * Nsl:].reshape(B * Nsl, kvw)], dim=0)
        if not cp.fused:
            full_t = g_text.new_zeros(P, B, Ll, kvw)
            full_s = g_text.new_zeros(P, B, max(Nsl, 1), kvw)
            for owner, lo, n in cp.text_sources(halo):
                off = (owner * Ll + lo) - (r * Ll - halo)
                full_t[owner, :, lo:lo + n] = g_text[:, off:off + n]
            for p in range(r):
                full_s[p, :, :Nsl] = g_sum[:, p * Nsl:(p + 1) * Nsl]
            dist.all_reduce(full_t, group=cp.group)
            dist.all_reduce(full_s, group=cp.group)
            g_local = g_local.clone()
            g_local[:B * Ll] += full_t[r].reshape(B * Ll, kvw)
            if Nsl > 0:
                g_local[B * Ll:] += full_s[r, :, :Nsl].reshape(B * Nsl, kvw)
            return g_local, None, None, None
        e = cp.counter_bwd
        cp.counter_bwd += 1
        slot = 2 + e % 2
        item = g_text.element_size()
        row_b = kvw * item
        base = 2 * cp.slot_bytes + (e % 2) * cp.ret_slot_bytes
        if cp.slot_last[slot] is not None:
            cp.consumed.wait_local(slot * P, P, None, cp.slot_last[slot] + 1)
        cp.slot_last[slot] = e
        # publish what belongs to others: [B x halo text rows | B x r*Nsl summary rows]
        n_pub = B * halo + B * r * Nsl
        if n_pub * row_b > cp.ret_slot_bytes:
            raise ValueError("context-parallel gradient return block exceeds the exchange buffer; build CpContext with "
                             "full_layers=True or a larger max_window")
        if n_pub > 0:
            pub = torch.cat([g_text[:, :halo].reshape(B * halo, kvw), g_sum[:, :r * Nsl].reshape(B * r * Nsl, kvw)], dim=0)
            cp.xbuf.view(cp.dtype, base, pub.numel()).copy_(pub.reshape(-1))
        cp.ready.set_on_all(slot * P + r, None, e + 1)
        # collect what later ranks computed for my rows
        for q in range(r + 1, P):
            halo_q = ctx.halo_of(q)
            start_q = q * Ll - halo_q                       # global text index of q's first halo row
            lo_g, hi_g = max(start_q, r * Ll), min(q * Ll, (r + 1) * Ll)
            flag = cp.ready.local_ptr(slot * P + q)
            if hi_g > lo_g:
                for b in range(B):
                    src = cp.xbuf.peer_ptrs[q] + base + (b * halo_q + (lo_g - start_q)) * row_b
                    _lib.call("ksa_peer_add_bf16", g_local[b * Ll + (lo_g - r * Ll):b * Ll + (hi_g - r * Ll)], src,
                              (hi_g - lo_g) * kvw, flag, None, e + 1, 16)
            if Nsl > 0:
                for b in range(B):
                    src = cp.xbuf.peer_ptrs[q] + base + (B * halo_q + b * q * Nsl + r * Nsl) * row_b
                    _lib.call("ksa_peer_add_bf16", g_local[B * Ll + b * Nsl:B * Ll + (b + 1) * Nsl], src, Nsl * kvw, flag,
                              None, e + 1, 8)
        cp.consumed.set_on_all(slot * P + r, None, e + 1)
        return g_local, None, None, None


def _ptr_array(values):
    import ctypes
    return (ctypes.c_void_p * len(values))(*[v if v else None for v in values])


def direct_exchange_possible(cp: CpContext, qkv: torch.Tensor, D: int, window_chunks: Optional[int]) -> bool:
    """Whether the attention kernels can read this layer's peer tiles in place (see the module docstring)."""
    sh = cp.shape
    return (cp.fused and qkv.is_cuda and D == 128 and window_chunks is not None and not ops.is_deterministic()
            and cp.size <= 8 and sh.local_sum % 128 == 0 and (window_chunks * sh.chunk) % 128 == 0
            and window_chunks * sh.chunk <= min(sh.local_len, cp.d_halo_max))


class _CpDirectAttention(torch.autograd.Function):
    """Summary-attention layer of one context-parallel shard with the exchange inside the attention kernels."""

    @staticmethod
    def _sources(cp: CpContext, base: int, slot: int, halo: int):
        sh, B, P, r = cp.shape, cp.batch, cp.size, cp.rank
        Ll, Nsl, kvw = sh.local_len, sh.local_sum, cp.kv_width
        row_b = kvw * 2
        ptr = cp.dbuf.peer_ptrs
        text = [ptr[r - 1] + base + (Ll - halo) * row_b if halo > 0 else 0, ptr[r] + base]
        text_flags = [cp.dready.local_ptr(slot * P + r - 1) if halo > 0 else 0, 0]
        sums = [ptr[p] + base + B * Ll * row_b for p in range(r + 1)]
        sum_flags = [cp.dready.local_ptr(slot * P + p) for p in range(r)] + [0]
        return _ptr_array(text), _ptr_array(text_flags), _ptr_array(sums), _ptr_array(sum_flags)

    @staticmethod
    def _publish(cp: CpContext, kv: torch.Tensor, slot: int, e: int):
        """Copy this rank's K|V rows into exchange slot ``slot`` and tell every rank (exchange number ``e``)."""
        P, r = cp.size, cp.rank
        if cp.d_slot_last[slot] is not None:      # every reader of the slot's previous contents is done
            cp.dconsumed.wait_local(slot * P, P, None, cp.d_slot_last[slot] + 1)
        cp.d_slot_last[slot] = e
        base = slot * cp.slot_bytes
        cp.dbuf.view(cp.dtype, base, kv.shape[0] * kv.shape[1]).view(kv.shape).copy_(kv)
        cp.dready.set_on_all(slot * P + r, None, e + 1)
        return base

    @staticmethod
    def forward(ctx, qkv, cp: CpContext, Hq, Hkv, D, window_chunks, scale):
        sh, B, P, r = cp.shape, cp.batch, cp.size, cp.rank
        Ll, Nsl, kvw = sh.local_len, sh.local_sum, cp.kv_width
        halo = sh.halo_len(window_chunks)
        e = cp.d_fwd
        cp.d_fwd += 1
        slot = e % 2
        base = _CpDirectAttention._publish(cp, qkv[:, Hq * D:], slot, e)
        text, text_flags, sums, sum_flags = _CpDirectAttention._sources(cp, base, slot, halo)
        rs = qkv.stride(0)
        out = torch.empty((B * (Ll + Nsl), Hq * D), dtype=qkv.dtype, device=qkv.device)
        lse = torch.empty((B, Hq, Ll), dtype=torch.float32, device=qkv.device)
        _lib.call("ksa_attn_fwd_cp", qkv, out, lse, B, Hq, Hkv, D, Ll, rs, Ll * rs, Hq * D, Ll * Hq * D,
                  text, halo, Ll, sums, r + 1, Nsl, kvw, Ll * kvw, Nsl * kvw, text_flags, sum_flags, e + 1,
                  r * Ll, r * Ll - halo, sh.chunk, sh.n_sum, window_chunks, 0, float(scale))
        # summary queries see their own chunk's text and summaries only: all local
        q, k, v = ops._packed_views(qkv, B, Ll, Hq, Hkv, D, 0)
        qs, ks, vs = ops._packed_views(qkv, B, Nsl, Hq, Hkv, D, B * Ll)
        os_ = out[B * Ll:].view(B, Nsl, Hq, D)
        lse_s = torch.empty((B, Hq, Nsl), dtype=torch.float32, device=qkv.device)
        _lib.call("ksa_summary_attn_fwd", qs, k, v, ks, vs, os_, lse_s, B, Hq, Hkv, D, Nsl, sh.seq_len,
                  rs, Nsl * rs, rs, Ll * rs, rs, Ll * rs, rs, Nsl * rs, rs, Nsl * rs, Hq * D, Nsl * Hq * D,
                  sh.chunk, sh.n_sum, r * sh.local_chunks, r * Ll, r * Nsl, float(scale))
        cp.dconsumed.set_on_all(slot * P + r, None, e + 1)
        ctx.save_for_backward(qkv, out, lse, lse_s)
        ctx.cfg = (cp, Hq, Hkv, D, window_chunks, scale, halo)
        return out

    @staticmethod
    def backward(ctx, dout):
        qkv, out, lse, lse_s = ctx.saved_tensors
        cp, Hq, Hkv, D, window_chunks, scale, halo = ctx.cfg
        sh, B, P, r = cp.shape, cp.batch, cp.size, cp.rank
        Ll, Nsl, kvw = sh.local_len, sh.local_sum, cp.kv_width
        dout = dout if dout.is_contiguous() else dout.contiguous()
        e = cp.d_bwd
        cp.d_bwd += 1
        slot, rslot = 2 + e % 2, 4 + e % 2
        base = _CpDirectAttention._publish(cp, qkv[:, Hq * D:], slot, e)
        text, text_flags, sums, sum_flags = _CpDirectAttention._sources(cp, base, slot, halo)
        # the owners' return blocks of this parity were last used two exchanges ago: they must have been folded
        if cp.d_slot_last[rslot] is not None:
            cp.dconsumed.wait_local(rslot * P, P, None, cp.d_slot_last[rslot] + 1)
        cp.d_slot_last[rslot] = e
        ret_base = 4 * cp.slot_bytes + (e % 2) * cp.d_ret_bytes
        H = cp.d_halo_max
        ret_sum_off = ret_base + B * H * kvw * 4
        ret_text = cp.dbuf.peer_ptrs[r - 1] + ret_base if halo > 0 else None
        ret_sum = _ptr_array([cp.dbuf.peer_ptrs[p] + ret_sum_off for p in range(r)] + [0])
        rs = qkv.stride(0)
        dqkv = torch.empty_like(qkv)
        drs = dqkv.stride(0)
        dq, dk, dv = ops._packed_views(dqkv, B, Ll, Hq, Hkv, D, 0)
        dqs, dks, dvs = ops._packed_views(dqkv, B, Nsl, Hq, Hkv, D, B * Ll)
        o = out[:B * Ll].view(B, Ll, Hq, D)
        do = dout[:B * Ll].view(B, Ll, Hq, D)
        lq_pad = (Ll + 127) // 128 * 128
        stats = torch.empty((2, B, Hq, lq_pad), dtype=torch.float32, device=qkv.device)
        dq32 = torch.empty((B, Ll, Hq, D), dtype=torch.float32, device=qkv.device)
        Ns = (r + 1) * Nsl
        part_k = part_v = None
        if _lib.attn_bwd_num_segments(Ll) > 1:
            part_k = torch.zeros((B, Ns, Hkv, D), dtype=torch.float32, device=qkv.device)
            part_v = torch.zeros_like(part_k)
        _lib.call("ksa_attn_bwd_fused_cp", qkv, o, do, lse, stats, dq32, dq, dk, dv, dks, dvs, B, Hq, Hkv, D, Ll,
                  rs, Ll * rs, Hq * D, Ll * Hq * D, drs, Ll * drs, drs, Ll * drs, drs, Ll * drs, drs, Nsl * drs, drs,
                  Nsl * drs, text, halo, Ll, sums, r + 1, Nsl, kvw, Ll * kvw, Nsl * kvw, text_flags, sum_flags, e + 1,
                  ret_text, ret_sum, kvw, H * kvw, Nsl * kvw, r * Ll, r * Ll - halo, sh.chunk, sh.n_sum, window_chunks, 0,
                  float(scale), part_k, part_v)
        cp.dready.set_on_all(rslot * P + r, None, e + 1)       # my additions to every owner's return block are done
        q, k, v = ops._packed_views(qkv, B, Ll, Hq, Hkv, D, 0)
        qs, ks, vs = ops._packed_views(qkv, B, Nsl, Hq, Hkv, D, B * Ll)
        os_ = out[B * Ll:].view(B, Nsl, Hq, D)
        dos = dout[B * Ll:].view(B, Nsl, Hq, D)
        own = r * Nsl * Hkv * D     # this rank's rows of the fp32 partial sums
        _lib.call("ksa_summary_attn_bwd", qs, k, v, ks, vs, os_, dos, lse_s, dqs, dk, dv, dks, dvs,
                  B, Hq, Hkv, D, Nsl, sh.seq_len, rs, Nsl * rs, rs, Ll * rs, rs, Ll * rs, rs, Nsl * rs, rs, Nsl * rs,
                  Hq * D, Nsl * Hq * D, drs, Nsl * drs, drs, Ll * drs, drs, Ll * drs, drs, Nsl * drs, drs, Nsl * drs,
                  sh.chunk, sh.n_sum, r * sh.local_chunks, r * Ll, r * Nsl, float(scale),
                  part_k.view(-1)[own:] if part_k is not None else None,
                  part_v.view(-1)[own:] if part_v is not None else None, Ns)
        if r < P - 1:     # what the later ranks computed for my last W*C text rows and for my summaries
            flags = cp.dready.local_ptr(rslot * P + r + 1)
            my_ret = cp.dbuf.local_ptr + ret_base
            h_next = min((r + 1) * Ll, window_chunks * sh.chunk)
            _lib.call("ksa_cp_fold_return", dqkv[Ll - h_next:, Hq * D:], my_ret, B, h_next, kvw, drs, Ll * drs, kvw,
                      H * kvw, flags, P - 1 - r, e + 1)
            _lib.call("ksa_cp_fold_return", dqkv[B * Ll:, Hq * D:], my_ret + B * H * kvw * 4, B, Nsl, kvw, drs, Nsl * drs,
                      kvw, Nsl * kvw, flags, P - 1 - r, e + 1)
        cp.dconsumed.set_on_all(rslot * P + r, None, e + 1)
        cp.dconsumed.set_on_all(slot * P + r, None, e + 1)
        return dqkv, None, None, None, None, None, None


# ------------------------------------------------------------------------------------------ sequence <-> head resharding
def _a2a(cp: CpContext, x: torch.Tensor, to_heads: bool, groups, total_width: int) -> torch.Tensor:
    """All-to-all between the sequence-sharded layout ``[B*Ll, total_width]`` (all columns of this rank's rows) and the
    head-sharded layout ``[B*L, w]`` (this rank's column groups of every row).  ``groups(rank)`` lists the
    ``(first column, width)`` ranges owned by ``rank`` in the full width.

    GPUs: every rank copies its block into a symmetric slot, raises its flag, and pulls what it needs from every peer
    with 2-D P2P copies (``ksa_peer_copy2d``) that wait, bounded, on the owner's flag.  CPU ranks: ``all_gather``.
    """
    sh, B, P, r = cp.shape, cp.batch, cp.size, cp.rank
    Ll, L = sh.local_len, sh.seq_len
    w = sum(g[1] for g in groups(r))
    x = x.contiguous()
    if to_heads:
        out = x.new_empty(B * L, w)
    else:
        out = x.new_empty(B * Ll, total_width)
    if not cp.fused:
        parts = [torch.empty_like(x) for _ in range(P)]
        dist.all_gather(parts, x, group=cp.group)
        for p in range(P):
            if to_heads:
                src = parts[p].view(B, Ll, total_width)
                off = 0
                for c0, cw in groups(r):
                    out.view(B, L, w)[:, p * Ll:(p + 1) * Ll, off:off + cw] = src[:, :, c0:c0 + cw]
                    off += cw
            else:
                src = parts[p].view(B, L, w)
                off = 0
                for c0, cw in groups(p):
                    out.view(B, Ll, total_width)[:, :, c0:c0 + cw] = src[:, r * Ll:(r + 1) * Ll, off:off + cw]
                    off += cw
        return out
    n = cp.a2a_counter
    cp.a2a_counter += 1
    slot = n % 2
    item = x.element_size()
    if x.numel() * item > cp.a2a_slot_bytes:
        raise ValueError("all-to-all block exceeds the exchange buffer")
    if cp.a2a_slot_last[slot] is not None:
        cp.a2a_consumed.wait_local(slot * P, P, None, cp.a2a_slot_last[slot] + 1)
    cp.a2a_slot_last[slot] = n
    base = slot * cp.a2a_slot_bytes
    cp.a2a_buf.view(x.dtype, base, x.numel()).copy_(x.reshape(-1))
    cp.a2a_ready.set_on_all(slot * P + r, None, n + 1)
    for p in range(P):
        flag = cp.a2a_ready.local_ptr(slot * P + p)
        peer = cp.a2a_buf.peer_ptrs[p] + base
        for b in range(B):
            off = 0
            for c0, cw in (groups(r) if to_heads else groups(p)):
                if to_heads:    # peer p's rows (b, 0..Ll) x my columns -> my rows (b, p*Ll ..)
                    src = peer + ((b * Ll) * total_width + c0) * item
                    dst = out[b * L + p * Ll:b * L + (p + 1) * Ll, off:off + cw]
                    _lib.call("ksa_peer_copy2d", dst, w * item, src, total_width * item, Ll, cw * item, flag, None,
                              n + 1, 16)
                else:           # peer p's copy of my rows (b, r*Ll ..) x p's columns -> my rows x p's column ranges
                    src = peer + ((b * L + r * Ll) * w + off) * item
                    dst = out[b * Ll:(b + 1) * Ll, c0:c0 + cw]
                    _lib.call("ksa_peer_copy2d", dst, total_width * item, src, w * item, Ll, cw * item, flag, None,
                              n + 1, 16)
                off += cw
    cp.a2a_consumed.set_on_all(slot * P + r, None, n + 1)
    return out


class _SeqToHead(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, cp, groups, total_width):
        ctx.cp, ctx.groups, ctx.total_width = cp, groups, total_width
        return _a2a(cp, x, True, groups, total_width)

    @staticmethod
    def backward(ctx, g):
        return _a2a(ctx.cp, g, False, ctx.groups, ctx.total_width), None, None, None


class _HeadToSeq(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, cp, groups, total_width):
        ctx.cp, ctx.groups, ctx.total_width = cp, groups, total_width
        return _a2a(cp, x, False, groups, total_width)

    @staticmethod
    def backward(ctx, g):
        return _a2a(ctx.cp, g, True, ctx.groups, ctx.total_width), None, None, None


def cp_full_attention_ulysses(qkv: torch.Tensor, cp: CpContext, Hq: int, Hkv: int, D: int, tok_window: int = 0,
                              scale: Optional[float] = None) -> torch.Tensor:
    """Full causal attention of a context-parallel group with balanced work: reshard the packed, rotated projection
    rows from sequence shards to head shards, run whole-sequence causal attention on ``Hq/P`` heads, reshard the
    output back (the data movement of DeepSpeed-Ulysses, ``muse/training/parallel.py:211-335``, done with P2P copies
    instead of four NCCL all-to-alls)."""
    P, B, L = cp.size, cp.batch, cp.shape.seq_len
    hq, hkv = Hq // P, Hkv // P

    def qkv_groups(r):
        return [(r * hq * D, hq * D), (Hq * D + r * hkv * D, hkv * D), ((Hq + Hkv) * D + r * hkv * D, hkv * D)]

    def o_groups(r):
        return [(r * hq * D, hq * D)]
    heads = _SeqToHead.apply(qkv, cp, qkv_groups, (Hq + 2 * Hkv) * D)
    o = ops.attention_packed(heads, B, L, 0, hq, hkv, D, tok_window=tok_window, scale=scale)
    return _HeadToSeq.apply(o, cp, o_groups, Hq * D)


def _cpu_shard_attention(q_t, k_t, v_t, q_s, k_s, v_s, sh: CpShape, halo: int, window: Optional[int], tok_window: int,
                         scale: float):
    """Dense-mask fp32 attention of one shard: global masks sliced to the staged key ranges."""
    r, Ll, Nsl, L = sh.rank, sh.local_len, sh.local_sum, sh.seq_len
    n_rep = q_t.shape[2] // k_t.shape[2]
    q0, k0 = r * Ll, r * Ll - halo
    if q_s is None:
        qi = torch.arange(q0, q0 + Ll)[:, None]
        ki = torch.arange(k0, q0 + Ll)[None, :]
        mask = ki <= qi
        if tok_window and tok_window > 0:
            mask = mask & (qi - ki < tok_window)
        o, _ = ref._masked_attention(q_t, ref._expand_kv(k_t, n_rep), ref._expand_kv(v_t, n_rep), mask, scale)
        return o.to(q_t.dtype), None
    tt, ts, st, ss = two_stream_masks(L, sh.chunk, sh.n_sum, window)
    s0, s1 = r * Nsl, (r + 1) * Nsl
    k_all = torch.cat([ref._expand_kv(k_t, n_rep), ref._expand_kv(k_s, n_rep)], dim=1)
    v_all = torch.cat([ref._expand_kv(v_t, n_rep), ref._expand_kv(v_s, n_rep)], dim=1)
    m_t = torch.cat([tt[q0:q0 + Ll, k0:q0 + Ll], ts[q0:q0 + Ll, :s1]], dim=1)
    m_s = torch.cat([st[s0:s1, k0:q0 + Ll], ss[s0:s1, :s1]], dim=1)
    o_t, _ = ref._masked_attention(q_t, k_all, v_all, m_t, scale)
    o_s, _ = ref._masked_attention(q_s, k_all, v_all, m_s, scale)
    return o_t.to(q_t.dtype), o_s.to(q_s.dtype)


def cp_attention_packed(qkv: torch.Tensor, cp: CpContext, Hq: int, Hkv: int, D: int, window_chunks: Optional[int] = None,
                        summaries: bool = True, tok_window: int = 0, scale: Optional[float] = None) -> torch.Tensor:
    """Attention of one context-parallel shard on packed, rotated projection rows.

    ``qkv`` is ``[B*Ll (+ B*Nsl), (Hq+2Hkv)*D]``: the shard's text rows, then (summary layers) its summary rows.
    ``window_chunks=None`` with ``summaries=False`` is a full-attention layer (``tok_window`` optional).  Returns the
    attention output rows ``[rows, Hq*D]`` in the same order.
    """
    sh, B, r = cp.shape, cp.batch, cp.rank
    Ll = sh.local_len
    Nsl = sh.local_sum if summaries else 0
    n_text = B * Ll
    if not summaries and window_chunks is None and cp.full_layer_mode == "ulysses":
        return cp_full_attention_ulysses(qkv, cp, Hq, Hkv, D, tok_window, scale)
    if qkv.shape[0] != n_text + B * Nsl:
        raise ValueError(f"expected {n_text + B * Nsl} packed rows for this shard, got {qkv.shape[0]}")
    scale = scale if scale is not None else D ** -0.5
    if summaries and direct_exchange_possible(cp, qkv, D, window_chunks):
        return _CpDirectAttention.apply(qkv, cp, Hq, Hkv, D, window_chunks, scale)
    kv = qkv[:, Hq * D:].contiguous()
    st_text, st_sum = _CpStage.apply(kv, cp, window_chunks, summaries)
    halo = sh.halo_len(window_chunks)
    q_t = qkv[:n_text, :Hq * D].view(B, Ll, Hq, D)
    k_t = st_text[..., :Hkv * D].view(B, halo + Ll, Hkv, D)
    v_t = st_text[..., Hkv * D:].view(B, halo + Ll, Hkv, D)
    q_s = k_s = v_s = None
    if summaries:
        q_s = qkv[n_text:, :Hq * D].view(B, Nsl, Hq, D)
        k_s = st_sum[..., :Hkv * D].view(B, (r + 1) * Nsl, Hkv, D)
        v_s = st_sum[..., Hkv * D:].view(B, (r + 1) * Nsl, Hkv, D)
    if not cp.fused:
        o_t, o_s = _cpu_shard_attention(q_t, k_t, v_t, q_s, k_s, v_s, sh, halo, window_chunks, tok_window, scale)
    elif summaries:
        o_t, o_s = ops.ksa_attention(q_t, k_t, v_t, q_s, k_s, v_s, sh.chunk, sh.n_sum, window_chunks, scale,
                                     q_off=r * Ll, k_off=r * Ll - halo, s_off=0, seq_len=sh.seq_len)
    else:
        o_t, o_s = ops.shard_causal_attention(q_t, k_t, v_t, scale, tok_window, q_off=r * Ll, k_off=r * Ll - halo,
                                              seq_len=sh.seq_len), None
    out = o_t.reshape(n_text, Hq * D)
    if o_s is not None:
        out = torch.cat([out, o_s.reshape(B * Nsl, Hq * D)], dim=0)
    return out


def shard_inputs(tokens: torch.Tensor, labels: Optional[torch.Tensor], rank: int, size: int):
    """This rank's contiguous slice of ``[B, L]`` tokens/labels (``muse/training/parallel.py:431-468`` splits the
    batch the same way for Ulysses)."""
    L = tokens.shape[1]
    Ll = L // size
    sl = slice(rank * Ll, (rank + 1) * Ll)
    return tokens[:, sl].contiguous(), (labels[:, sl].contiguous() if labels is not None else None)
