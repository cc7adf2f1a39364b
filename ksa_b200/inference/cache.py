"""Contiguous ring-buffer KV cache for Kwai Summary Attention decoding, batched, with device-resident metadata.

Per summary-attention layer one K and one V tensor ``[B, Hkv, cap, D]`` laid out as

    [ scratch (S) | current chunk (C, filled right -> left) | sliding-chunk ring (W*C) | summaries (append) ]

following ``examples/pretrain/hf_template/modeling_qwen3sa.py:85-505``.  Keys are cached after RoPE, so physical
order is irrelevant and every query attends ONE contiguous slice with no mask:

* text token at chunk offset ``cbl`` (tokens already in the chunk): written at slot ``S + C - 1 - cbl``; attends
  ``[S + C - 1 - cbl, S + C + ring_valid)`` while fewer than ``W`` chunks have been flushed, and
  ``[S + C - 1 - cbl, S + C + W*C + n_sum - W*S)`` afterwards - the newest ``W*S`` summaries (those of the chunks
  still inside the window) sit at the tail of the summary region and are cut off by the slice end;
* at a chunk boundary the step carries ``1 + S`` queries: the last text token as above, and summary token ``j``
  written to scratch slot ``S - 1 - j`` attending ``[S - 1 - j, S + C)`` (its own chunk's text and the summaries up
  to itself: causal for any ``S``; the reference's boundary attention is non-causal over the summaries and thus
  exact only for ``S = 1``); afterwards the chunk's ``C`` text rows are copied into ring slot ``(chunk mod W) * C``
  and the ``S`` summary rows are appended to the summary region.
* full-attention layers of a hybrid stack keep an append-only text cache and never store summaries.

Unlike the reference (batch 1 only, Python-side counters), every counter here is a ``[B]`` int32 device tensor, so
sequences of one batch may sit at different chunk phases and a step is a fixed sequence of kernel launches.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Tuple

import torch


@dataclass
class CacheSpec:
    chunk: int        # C
    n_sum: int        # S
    window: int       # W (chunks)
    max_chunks: int   # summaries the buffer can hold = max_chunks * S

    @property
    def ring(self) -> int:
        return self.window * self.chunk

    @property
    def capacity(self) -> int:
        return self.n_sum + self.chunk + self.ring + self.max_chunks * self.n_sum

    @property
    def text0(self) -> int:      # first slot after the current-chunk region
        return self.n_sum + self.chunk

    @property
    def sum0(self) -> int:       # first slot of the summary region
        return self.n_sum + self.chunk + self.ring


class KsaLayerCache:
    """Ring-buffer cache of one summary-attention layer."""

    def __init__(self, spec: CacheSpec, batch: int, n_kv_heads: int, head_dim: int, dtype, device):
        self.spec = spec
        self.k = torch.zeros(batch, n_kv_heads, spec.capacity, head_dim, dtype=dtype, device=device)
        self.v = torch.zeros_like(self.k)


class FullLayerCache:
    """Append-only text cache of one full-attention layer."""

    def __init__(self, max_len: int, batch: int, n_kv_heads: int, head_dim: int, dtype, device):
        self.k = torch.zeros(batch, n_kv_heads, max_len, head_dim, dtype=dtype, device=device)
        self.v = torch.zeros_like(self.k)
        self.max_len = max_len


class CacheState:
    """Per-sequence counters shared by all layers (they advance in lock step): text length, chunk phase, chunks done."""

    def __init__(self, batch: int, device):
        z = lambda: torch.zeros(batch, dtype=torch.int32, device=device)
        self.text_len = z()      # text tokens written so far
        self.cbl = z()           # tokens in the current (unfinished) chunk
        self.chunks = z()        # chunks flushed so far (= summaries groups stored)

    def clone(self) -> "CacheState":
        c = CacheState.__new__(CacheState)
        c.text_len, c.cbl, c.chunks = self.text_len.clone(), self.cbl.clone(), self.chunks.clone()
        return c


def text_step_slices(spec: CacheSpec, st: CacheState) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """For the next text token of every sequence: (write slot, slice start, slice length) on the ring-buffer cache."""
    S, C, W = spec.n_sum, spec.chunk, spec.window
    slot = (S + C - 1) - st.cbl
    ring_valid = torch.clamp(st.chunks, max=W) * C
    old_summaries = torch.clamp(st.chunks - W, min=0) * S
    full = st.chunks >= W
    end = torch.where(full, spec.sum0 + old_summaries, spec.text0 + ring_valid)
    return slot, slot, (end - slot)


def summary_step_slices(spec: CacheSpec, batch: int, device) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """For the S summary tokens of a boundary step: (write slots, starts, lengths), each ``[B, S]``."""
    S, C = spec.n_sum, spec.chunk
    j = torch.arange(S, dtype=torch.int32, device=device)
    slot = (S - 1 - j).unsqueeze(0).expand(batch, S).contiguous()
    return slot, slot, (S + C - slot)


def flush_plan(spec: CacheSpec, st: CacheState) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
    """Moves after a boundary step: chunk text ``[S, S+C)`` -> ring slot, scratch ``[0, S)`` -> summary region.

    Scratch holds summary j at slot S-1-j; the summary region is append-only and order-free (keys carry their RoPE),
    so the S rows move as one block.
    """
    S, C, W = spec.n_sum, spec.chunk, spec.window
    B = st.chunks.shape[0]
    dev = st.chunks.device
    src_text = torch.full((B,), S, dtype=torch.int32, device=dev)
    dst_text = spec.text0 + (st.chunks % max(W, 1)) * C
    src_sum = torch.zeros(B, dtype=torch.int32, device=dev)
    dst_sum = spec.sum0 + st.chunks * S
    return src_text, dst_text, src_sum, dst_sum
