"""Attention back ends: an eager masked softmax and the tensor-core kernel (causal, token sliding window), the
counterparts of ``EagerAttention`` / ``FlashAttention2`` (``muse/layers/attention_utils.py:76-167,169-249,252-259``).

Inputs are ``[b, s, n_heads, d]`` (queries) and ``[b, s_kv, n_kv_heads, d]``; grouped-query heads are expanded inside
the back end, never by the caller.
"""
import math
from typing import Dict, Optional

import torch
from torch import nn

from .. import ops
from ..ops import reference as ref


class EagerAttention(nn.Module):
    """Dense softmax attention; ``mask`` ``[b|1, s, s_kv]`` bool (``True`` = attend) or causal when ``None``."""

    def forward(self, q, k, v, mask: Optional[torch.Tensor] = None, is_causal: bool = True,
                scale: Optional[float] = None, window: int = -1, cu_seqlens: Optional[torch.Tensor] = None):
        scale = scale if scale is not None else 1.0 / math.sqrt(q.shape[-1])
        if mask is None and is_causal:
            return ref.causal_attention(q, k, v, scale, window, cu_seqlens)
        n_rep = q.shape[2] // k.shape[2]
        kf, vf = ref._expand_kv(k, n_rep), ref._expand_kv(v, n_rep)
        if mask is None:
            mask = torch.ones(q.shape[1], k.shape[1], dtype=torch.bool, device=q.device)
        outs = []
        for b in range(q.shape[0]):
            m = mask if mask.dim() == 2 else mask[b if mask.shape[0] > 1 else 0]
            o, _ = ref._masked_attention(q[b:b + 1], kf[b:b + 1], vf[b:b + 1], m, scale)
            outs.append(o)
        return torch.cat(outs, dim=0).to(q.dtype)


class TensorCoreAttention(nn.Module):
    """Causal attention on the tcgen05 kernel (``window > 0`` keeps keys with ``q - k < window``; ``cu_seqlens``:
    documents packed into one sequence, as ``flash_attn_varlen_func`` takes them in the reference,
    ``muse/layers/attention_utils.py:195-246``).  Arbitrary masks fall back to the eager form."""

    def __init__(self):
        super().__init__()
        self.eager = EagerAttention()

    def forward(self, q, k, v, mask: Optional[torch.Tensor] = None, is_causal: bool = True,
                scale: Optional[float] = None, window: int = -1, cu_seqlens: Optional[torch.Tensor] = None):
        fast = q.is_cuda and q.dtype == torch.bfloat16 and mask is None and is_causal and q.shape[-1] in (64, 128)
        if not fast:
            return self.eager(q, k, v, mask, is_causal, scale, window, cu_seqlens)
        return ops.causal_attention(q, k, v, scale, window, cu_seqlens=cu_seqlens)


ATTENTION_BACKENDS: Dict[str, type] = {"eager": EagerAttention, "tensor_core": TensorCoreAttention,
                                       "flash_attention_2": TensorCoreAttention}


def get_attention_backend(name: str) -> nn.Module:
    """``flash_attention_2`` is accepted as an alias so that the reference's configs load unchanged."""
    if name not in ATTENTION_BACKENDS:
        raise KeyError(f"unknown attention backend {name!r}; have {sorted(ATTENTION_BACKENDS)}")
    return ATTENTION_BACKENDS[name]()
