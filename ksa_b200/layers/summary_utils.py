"""Summary batch builder: the interleaved (expanded) form of a batch with summary tokens after every chunk
(``muse/layers/summary_utils.py:19-221``, ``muse/layers/summary_context.py:111-170``).

The training path of this package keeps text and summary rows in two streams and never builds the expanded sequence;
this builder exists for code that wants the reference's representation (data inspection, the HF template, tests).  It
is fully vectorised: one ``SummaryLayout`` gives the row indices, position ids and the summary mask.
"""
from dataclasses import dataclass
from typing import Optional

import torch

from ..ops.layout import SummaryLayout, get_layout


@dataclass
class SummaryBatch:
    input_ids: torch.Tensor          # [B, L + Ns] text tokens with the summary token ids inserted after every chunk
    summary_mask: torch.Tensor       # [L + Ns] bool, True on summary positions
    position_ids: torch.Tensor       # [B, L + Ns]
    cu_seqlens: Optional[torch.Tensor]   # document boundaries in expanded coordinates
    layout: SummaryLayout
    labels: Optional[torch.Tensor] = None      # stay at the original length (the decoder drops summary rows)
    loss_mask: Optional[torch.Tensor] = None


def build_summary_batch(input_ids: torch.Tensor, chunk: int, n_sum: int, summary_token_begin: int,
                        text_pos_type: str = "origin", sum_pos_type: str = "last_chunk_slice_right",
                        cu_seqlens: Optional[torch.Tensor] = None, labels: Optional[torch.Tensor] = None,
                        loss_mask: Optional[torch.Tensor] = None) -> SummaryBatch:
    """``input_ids`` ``[B, L]`` -> :class:`SummaryBatch`; summary token ``j`` of a chunk has id ``begin + j``."""
    B, L = input_ids.shape
    dev = input_ids.device
    layout = get_layout(L, chunk, n_sum, text_pos_type, sum_pos_type)
    sum_ids = (summary_token_begin + torch.arange(n_sum, device=dev)).repeat(layout.n_chunks)
    expanded = layout.interleave(input_ids, sum_ids[None].expand(B, -1).to(input_ids.dtype), dim=1)
    pos = layout.expanded_position_ids(dev)[None].expand(B, -1)
    return SummaryBatch(expanded, layout.summary_mask_expanded(dev), pos,
                        layout.remap_cu_seqlens(cu_seqlens) if cu_seqlens is not None else None, layout, labels, loss_mask)
