"""Closed-form sequence layout for Kwai Summary Attention.

A text sequence of length ``L`` is cut into chunks of ``C`` tokens and ``S``
summary tokens follow each chunk.  The reference materialises this as one
interleaved sequence of length ``L + ceil(L/C)*S`` with a Python loop per chunk
(``muse/layers/summary_utils.py:19-221``).  Here text rows and summary rows are
two separate streams and everything that depends only on ``(L, C, S)`` —
position ids, the interleaved<->two-stream index maps, the remapped
``cu_seqlens`` — is computed in closed form, once per shape, with no host sync.
"""
from __future__ import annotations

from dataclasses import dataclass
from functools import lru_cache
from typing import Optional, Tuple

import torch


@dataclass(frozen=True)
class SummaryLayout:
    seq_len: int              # L, text tokens
    chunk: int                # C
    n_sum: int                # S
    text_pos_type: str = "origin"
    sum_pos_type: str = "last_chunk_slice_right"
    drop_partial: bool = False  # True: a trailing partial chunk gets no summary tokens (prefill / decoding)

    @property
    def n_chunks(self) -> int:
        if self.drop_partial:
            return self.seq_len // self.chunk
        return (self.seq_len + self.chunk - 1) // self.chunk

    @property
    def n_summary_rows(self) -> int:
        return self.n_chunks * self.n_sum

    @property
    def expanded_len(self) -> int:
        return self.seq_len + self.n_summary_rows

    # ---- position ids ----------------------------------------------------
    def text_position_ids(self, device=None) -> torch.Tensor:
        t = torch.arange(self.seq_len, device=device, dtype=torch.long)
        if self.text_pos_type == "origin":
            return t
        if self.text_pos_type == "inner_chunk":
            return t % self.chunk
        raise ValueError(f"unknown summary_chunk_position_ids_type {self.text_pos_type!r}")

    def summary_position_ids(self, device=None) -> torch.Tensor:
        """Position id of summary token ``j`` of chunk ``i`` (row ``i*S + j``).

        ``last_chunk_slice_right``: the chunk's text range is cut into ``S``
        slices and token ``j`` takes the last position of slice ``j``; for
        ``S = 1`` that is the chunk's last text position.  The reference derives
        the chunk start from the *current* chunk's length
        (``muse/layers/summary_utils.py:148``), which only differs for a ragged
        last chunk; the chunk's true start ``i*C`` is used here.
        """
        i = torch.arange(self.n_chunks, device=device, dtype=torch.long).repeat_interleave(self.n_sum)
        j = torch.arange(self.n_sum, device=device, dtype=torch.long).repeat(self.n_chunks)
        if self.sum_pos_type == "zeros":
            return torch.zeros_like(i)
        start = i * self.chunk
        end = torch.clamp((i + 1) * self.chunk, max=self.seq_len)
        length = end - start
        if self.sum_pos_type == "last_chunk_slice_right":
            pos = start + ((j + 1) * length) // self.n_sum - 1
        elif self.sum_pos_type == "last_chunk_slice_left":
            pos = start + (j * length) // self.n_sum - 1
        else:
            raise ValueError(f"unknown summary_token_position_ids_type {self.sum_pos_type!r}")
        return torch.maximum(pos, start)

    # ---- interleaved <-> two-stream index maps ---------------------------
    def text_rows_in_expanded(self, device=None) -> torch.Tensor:
        t = torch.arange(self.seq_len, device=device, dtype=torch.long)
        return t + (t // self.chunk) * self.n_sum

    def summary_rows_in_expanded(self, device=None) -> torch.Tensor:
        i = torch.arange(self.n_chunks, device=device, dtype=torch.long).repeat_interleave(self.n_sum)
        j = torch.arange(self.n_sum, device=device, dtype=torch.long).repeat(self.n_chunks)
        end = torch.clamp((i + 1) * self.chunk, max=self.seq_len)
        return end + i * self.n_sum + j

    def summary_mask_expanded(self, device=None) -> torch.Tensor:
        m = torch.zeros(self.expanded_len, dtype=torch.bool, device=device)
        m[self.summary_rows_in_expanded(device)] = True
        return m

    def expanded_position_ids(self, device=None) -> torch.Tensor:
        out = torch.empty(self.expanded_len, dtype=torch.long, device=device)
        out[self.text_rows_in_expanded(device)] = self.text_position_ids(device)
        out[self.summary_rows_in_expanded(device)] = self.summary_position_ids(device)
        return out

    def interleave(self, text: torch.Tensor, summary: torch.Tensor, dim: int = 1) -> torch.Tensor:
        """Two streams -> the reference's interleaved sequence along ``dim``."""
        shape = list(text.shape)
        shape[dim] = self.expanded_len
        out = text.new_empty(shape)
        out.index_copy_(dim, self.text_rows_in_expanded(text.device), text)
        out.index_copy_(dim, self.summary_rows_in_expanded(text.device), summary)
        return out

    def split(self, expanded: torch.Tensor, dim: int = 1) -> Tuple[torch.Tensor, torch.Tensor]:
        return (expanded.index_select(dim, self.text_rows_in_expanded(expanded.device)),
                expanded.index_select(dim, self.summary_rows_in_expanded(expanded.device)))

    def remap_cu_seqlens(self, cu_seqlens: torch.Tensor) -> torch.Tensor:
        """Document boundaries in text coordinates -> expanded coordinates."""
        out = cu_seqlens + (cu_seqlens // self.chunk) * self.n_sum
        # the end of the sequence also closes a ragged last chunk, whose summary tokens follow it
        return torch.where(cu_seqlens >= self.seq_len, torch.full_like(out, self.expanded_len), out)


@lru_cache(maxsize=64)
def get_layout(seq_len: int, chunk: int, n_sum: int, text_pos_type: str = "origin",
               sum_pos_type: str = "last_chunk_slice_right", drop_partial: bool = False) -> SummaryLayout:
    return SummaryLayout(seq_len, chunk, n_sum, text_pos_type, sum_pos_type, drop_partial)


# --------------------------------------------------------------------------
# Mask semantics (True = may attend).
# --------------------------------------------------------------------------
def dense_interleaved_mask(expanded_len: int, chunk: int, n_sum: int, window: int,
                           device=None) -> torch.Tensor:
    """The KSA rule on the interleaved sequence, as one vectorised predicate.

    With ``blk = C + S``, ``qc = q // blk``, ``kc = k // blk``:
      * summary query: keys of its own chunk only, causal;
      * text query: causal and (text key with ``qc - kc <= W``  or  summary key
        with ``qc - kc > W``).
    Same truth table as ``muse/layers/summary_attention_func.py:506-584``.
    """
    blk = chunk + n_sum
    if expanded_len % blk != 0:
        raise ValueError(f"expanded length {expanded_len} is not a multiple of chunk+summary {blk}")
    idx = torch.arange(expanded_len, device=device)
    c = idx // blk
    is_sum = (idx % blk) >= chunk
    q, k = idx[:, None], idx[None, :]
    qc, kc = c[:, None], c[None, :]
    q_sum, k_sum = is_sum[:, None], is_sum[None, :]
    causal = k <= q
    sum_rule = q_sum & (qc == kc) & causal
    text_rule = (~q_sum) & causal & (((~k_sum) & (qc - kc <= window)) | (k_sum & (qc - kc > window)))
    return sum_rule | text_rule


def two_stream_masks(seq_len: int, chunk: int, n_sum: int, window: int, device=None,
                     q_offset: int = 0, q_len: Optional[int] = None, n_summary_rows: Optional[int] = None):
    """Masks of the two-stream formulation.

    Returns ``(tt, ts, st, ss)``: text-query x text-key, text-query x summary-key,
    summary-query x text-key, summary-query x summary-key.  ``q_offset``/``q_len``
    restrict the text queries to a slice (context-parallel shards).
    """
    n_chunks = (seq_len + chunk - 1) // chunk if n_summary_rows is None else n_summary_rows // max(n_sum, 1)
    q_len = seq_len - q_offset if q_len is None else q_len
    t = torch.arange(q_offset, q_offset + q_len, device=device)
    u = torch.arange(seq_len, device=device)
    s = torch.arange(n_chunks * n_sum, device=device)
    qc, kc, sc = (t // chunk)[:, None], (u // chunk)[None, :], (s // n_sum)
    tt = (u[None, :] <= t[:, None]) & (qc - kc <= window)
    ts = (qc - sc[None, :]) > window
    st = sc[:, None] == kc
    ss = (sc[:, None] == sc[None, :]) & ((s % n_sum)[None, :] <= (s % n_sum)[:, None])
    return tt, ts, st, ss


def count_attended_pairs(seq_len: int, chunk: int, n_sum: int, window: int) -> int:
    """Number of (query, key) pairs the KSA mask allows, per head (closed form)."""
    total = 0
    n_chunks = (seq_len + chunk - 1) // chunk
    for i in range(n_chunks):
        c = min(chunk, seq_len - i * chunk)
        in_window = min(i, window) * chunk
        old = max(0, i - window) * n_sum
        total += c * (in_window + old) + c * (c + 1) // 2
        total += n_sum * c + n_sum * (n_sum + 1) // 2
    return total
