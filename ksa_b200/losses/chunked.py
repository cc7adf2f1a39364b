"""Sequence-chunked lm_head + cross entropy (+ KL against a teacher) with bounded logits memory.

The reference needs this class for long sequences: it slices the hidden states into chunks of
``minibatch_size`` tokens, runs lm_head + CE (+ KL) per chunk with ``autograd.grad``, accumulates the gradient of
the hidden states, calls ``student_hidden.backward`` once and then adds the lm_head gradients by hand
(``muse/losses/chunked_distill_loss_computer.py:46-214``).  On GPUs the plain language-model loss does not need it
here - ``ops.linear_cross_entropy`` is already chunked and produces both gradients inside the forward pass - so this
class serves (a) the distillation mode, where the KL term needs both sets of logits per chunk, and (b) CPU runs.  It
keeps the reference's contract: ``forward_and_backward`` runs the backward pass itself and returns detached scalars.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch
import torch.nn.functional as F

from .. import ops


class ChunkedDistillLossComputer:
    def __init__(self, lm_head_weight: torch.Tensor, minibatch_size: int = 1024, lm_factor: float = 1.0,
                 kl_factor: float = 0.0, enable_kl: bool = False, ignore_index: int = -100):
        self.weight = lm_head_weight
        self.minibatch_size = int(minibatch_size)
        self.lm_factor, self.kl_factor, self.enable_kl = lm_factor, kl_factor, enable_kl
        self.ignore_index = ignore_index

    def forward_and_backward(self, student_hidden: torch.Tensor, teacher_hidden: Optional[torch.Tensor],
                             labels: torch.Tensor, gradient_accumulation_steps: int = 1,
                             extra_loss: Optional[torch.Tensor] = None) -> Dict[str, torch.Tensor]:
        """``student_hidden`` ``[B, L, D]`` (requires grad), ``labels`` ``[B, L]`` (already shifted)."""
        B, L, D = student_hidden.shape
        h = student_hidden.reshape(B * L, D)
        lab = labels.reshape(B * L)
        n_valid = (lab != self.ignore_index).sum().clamp(min=1)
        scale = 1.0 / gradient_accumulation_steps
        if not self.enable_kl or teacher_hidden is None:
            ce = ops.linear_cross_entropy(h, self.weight, lab, self.ignore_index, self.minibatch_size)
            total = self.lm_factor * ce + (extra_loss if extra_loss is not None else 0.0)
            (total * scale).backward()
            zero = torch.zeros((), device=h.device)
            return {"total_loss": total.detach(), "ce_loss": ce.detach(), "kl_loss": zero}
        # distillation: per chunk logits of student and teacher; gradients accumulate through autograd
        th = teacher_hidden.reshape(B * L, D).detach()
        grad_h = torch.zeros_like(h)
        ce_sum = torch.zeros((), device=h.device, dtype=torch.float32)
        kl_sum = torch.zeros((), device=h.device, dtype=torch.float32)
        w = self.weight
        w_grad = torch.zeros_like(w, dtype=torch.float32) if w.requires_grad else None
        w_used = False
        for s in range(0, B * L, self.minibatch_size):
            e = min(B * L, s + self.minibatch_size)
            hs = h[s:e].detach().requires_grad_(True)
            logits = ops.linear(hs, w).float()
            with torch.no_grad():
                t_logits = ops.linear(th[s:e], w).float()
            valid = lab[s:e] != self.ignore_index
            ce_c = F.cross_entropy(logits, lab[s:e], ignore_index=self.ignore_index, reduction="sum")
            logp = F.log_softmax(logits, -1)
            tp = F.softmax(t_logits, -1)
            kl_c = ((tp * (torch.log(tp.clamp_min(1e-20)) - logp)).sum(-1) * valid).sum()
            loss_c = (self.lm_factor * ce_c + self.kl_factor * kl_c) / n_valid * scale
            # a weight with an fp32 ``main_grad`` buffer gets its gradient written there by ops.linear's backward,
            # and autograd sees none for it (allow_unused)
            grads = torch.autograd.grad(loss_c, [hs] + ([w] if w_grad is not None else []), allow_unused=True)
            grad_h[s:e] = grads[0]
            if w_grad is not None and grads[1] is not None:
                w_grad += grads[1].float()
                w_used = True
            ce_sum += ce_c.detach()
            kl_sum += kl_c.detach()
        # The lm_head gradient goes in BEFORE the backward pass through the model: an engine that reduces and updates
        # a unit as soon as the backward pass has left it would otherwise miss it.
        if w_grad is not None and w_used:
            mg = getattr(w, "main_grad", None)
            if mg is not None:
                if getattr(w, "_grad_written", False):
                    mg.add_(w_grad)
                else:
                    mg.copy_(w_grad)
                    w._grad_written = True
            else:
                w.grad = w_grad.to(w.dtype) if w.grad is None else w.grad + w_grad.to(w.dtype)
        # one backward pass through the model for the hidden-state gradient and the extra (attention matching) loss
        roots, root_grads = [student_hidden], [grad_h.view(B, L, D)]
        if extra_loss is not None and extra_loss.requires_grad:
            roots.append(extra_loss * scale)
            root_grads.append(None)
        torch.autograd.backward(roots, root_grads)
        ce, kl = ce_sum / n_valid, kl_sum / n_valid
        total = self.lm_factor * ce + self.kl_factor * kl + (extra_loss.detach() if extra_loss is not None else 0.0)
        return {"total_loss": total, "ce_loss": ce, "kl_loss": kl}
