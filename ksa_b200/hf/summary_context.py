"""Layout helpers for the HF model: where summary tokens sit and which position ids they get.

Stand-alone (no dependency on the training package) so that the template works from a bare checkpoint directory;
the formulas are the closed forms of ``ksa_b200.ops.layout`` (a trailing partial chunk gets no summary tokens, as in
``examples/pretrain/hf_template/summary_context.py:17-133`` of the reference).
"""
from __future__ import annotations

from dataclasses import dataclass

import torch


@dataclass
class SummaryContext:
    seq_len: int
    chunk: int
    n_sum: int
    text_pos_type: str = "origin"
    sum_pos_type: str = "last_chunk_slice_right"

    @property
    def n_chunks(self) -> int:
        return self.seq_len // self.chunk

    @property
    def n_summary_rows(self) -> int:
        return self.n_chunks * self.n_sum

    def text_position_ids(self, device=None) -> torch.Tensor:
        t = torch.arange(self.seq_len, device=device)
        return t if self.text_pos_type == "origin" else t % self.chunk

    def summary_position_ids(self, device=None) -> torch.Tensor:
        i = torch.arange(self.n_chunks, device=device).repeat_interleave(self.n_sum)
        j = torch.arange(self.n_sum, device=device).repeat(self.n_chunks)
        if self.sum_pos_type == "zeros":
            return torch.zeros_like(i)
        start = i * self.chunk
        if self.sum_pos_type == "last_chunk_slice_right":
            pos = start + ((j + 1) * self.chunk) // self.n_sum - 1
        else:
            pos = start + (j * self.chunk) // self.n_sum - 1
        return torch.maximum(pos, start)

    def masks(self, window: int, device=None):
        """(text x text, text x summary, summary x text, summary x summary) boolean masks, True = may attend."""
        t = torch.arange(self.seq_len, device=device)
        s = torch.arange(self.n_summary_rows, device=device)
        qc, kc, sc = (t // self.chunk)[:, None], (t // self.chunk)[None, :], s // max(self.n_sum, 1)
        tt = (t[None, :] <= t[:, None]) & (qc - kc <= window)
        ts = (qc - sc[None, :]) > window
        st = sc[:, None] == kc
        ss = (sc[:, None] == sc[None, :]) & ((s % max(self.n_sum, 1))[None, :] <= (s % max(self.n_sum, 1))[:, None])
        return tt, ts, st, ss


def parse_pattern(value, n_layers: int):
    """An int, a list, or a pattern string such as ``"([1]*3+[0]*1)*7"`` -> list of ``n_layers`` ints (no eval)."""
    if isinstance(value, (list, tuple)):
        return [int(v) for v in value]
    if isinstance(value, int):
        return [value] * n_layers
    text = "".join(str(value).split())
    pos = 0

    def peek():
        return text[pos] if pos < len(text) else ""

    def integer():
        nonlocal pos
        a = pos
        while peek().isdigit():
            pos += 1
        if a == pos:
            raise ValueError(f"bad pattern {value!r}")
        return int(text[a:pos])

    def atom():
        nonlocal pos
        if peek() == "[":
            pos += 1
            vals = []
            while peek() != "]":
                vals.append(integer())
                if peek() == ",":
                    pos += 1
            pos += 1
            return vals
        if peek() == "(":
            pos += 1
            vals = expr()
            if peek() != ")":
                raise ValueError(f"bad pattern {value!r}")
            pos += 1
            return vals
        raise ValueError(f"bad pattern {value!r}")

    def term():
        nonlocal pos
        vals = atom()
        while peek() == "*":
            pos += 1
            vals = vals * integer()
        return vals

    def expr():
        nonlocal pos
        vals = term()
        while peek() == "+":
            pos += 1
            vals = vals + term()
        return vals

    out = expr()
    if pos != len(text):
        raise ValueError(f"bad pattern {value!r}")
    return out
