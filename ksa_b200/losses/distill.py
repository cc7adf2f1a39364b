"""Distillation losses between a summary-attention student and its full-attention teacher
(``muse/losses/distill.py:24-139``): per-layer attention-output MSE clamped to [0, 0.1], cosine distance, and the KL
divergence of student vs teacher logits."""
from __future__ import annotations

from typing import List, Optional

import torch
import torch.nn.functional as F


def attention_mse_loss(student: List[torch.Tensor], teacher: List[torch.Tensor], clamp_max: float = 0.1) -> torch.Tensor:
    """Mean over layers of ``clamp(mse(student_l, teacher_l), 0, clamp_max)``."""
    if not student:
        return torch.zeros(())
    per_layer = [F.mse_loss(s.float(), t.float().detach()).clamp(0.0, clamp_max) for s, t in zip(student, teacher)]
    return torch.stack(per_layer).mean()


def attention_cosine_loss(student: List[torch.Tensor], teacher: List[torch.Tensor]) -> torch.Tensor:
    """Mean over layers and tokens of ``1 - cos(student, teacher)``."""
    if not student:
        return torch.zeros(())
    per_layer = [(1.0 - F.cosine_similarity(s.float(), t.float().detach(), dim=-1)).mean() for s, t in zip(student, teacher)]
    return torch.stack(per_layer).mean()


def kl_divergence_loss(student_logits: torch.Tensor, teacher_logits: torch.Tensor, mask: Optional[torch.Tensor] = None,
                       temperature: float = 1.0) -> torch.Tensor:
    """``KL(teacher || student)`` per token (batchmean over valid tokens), fp32."""
    s = F.log_softmax(student_logits.float() / temperature, dim=-1)
    t = F.softmax(teacher_logits.float().detach() / temperature, dim=-1)
    kl = (t * (torch.log(t.clamp_min(1e-20)) - s)).sum(-1)
    if mask is not None:
        m = mask.to(kl.dtype).reshape(kl.shape)
        return (kl * m).sum() / m.sum().clamp(min=1) * temperature ** 2
    return kl.mean() * temperature ** 2


def rms_normalize(x: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    """RMS-normalise attention outputs before comparing them (``summary_distill_attention_norm``)."""
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)).to(x.dtype)
