"""Token cross entropy in fp32, mean over non-ignored tokens (``muse/losses/ce.py:32-140``)."""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F


class CrossEntropyLoss(nn.Module):
    """``shift_labels=True`` drops the last logit and the first label (callers that pass unshifted labels);
    the trainer passes labels that are already shifted and uses ``shift_labels=False``."""

    def __init__(self, ignore_index: int = -100, shift_labels: bool = False, reduction: str = "mean"):
        super().__init__()
        self.ignore_index, self.shift_labels, self.reduction = ignore_index, shift_labels, reduction

    def forward(self, logits: torch.Tensor, labels: torch.Tensor) -> torch.Tensor:
        if self.shift_labels:
            logits, labels = logits[..., :-1, :], labels[..., 1:]
        loss = F.cross_entropy(logits.float().reshape(-1, logits.shape[-1]), labels.reshape(-1),
                               ignore_index=self.ignore_index, reduction="none")
        if self.reduction == "none":
            return loss.view(labels.shape)
        valid = (labels.reshape(-1) != self.ignore_index).sum().clamp(min=1)
        return loss.sum() / valid if self.reduction == "mean" else loss.sum()
