"""Rotary position embeddings with an fp32 cos/sin cache indexed by position ids.

``RotaryPositionalEmbeddings`` pairs element ``i`` with ``i + d/2`` (HF "half split", what Qwen3 uses,
``muse/layers/position_embeddings.py:165-293``); ``LlamaRotaryPositionalEmbeddings`` pairs ``2i`` with ``2i + 1``
(``:48-162``).  The fused QK-norm + RoPE kernel of ``ksa_b200.ops`` computes the same angles on the fly; these modules
are the stand-alone form.
"""
from typing import Optional

import torch
from torch import nn


class _RopeBase(nn.Module):
    def __init__(self, dim: int, max_seq_len: int = 4096, base: float = 10000.0):
        super().__init__()
        if dim % 2:
            raise ValueError("rotary dimension must be even")
        self.dim, self.max_seq_len, self.base = dim, max_seq_len, base
        self.rope_init()

    def rope_init(self) -> None:
        theta = 1.0 / (self.base ** (torch.arange(0, self.dim, 2, dtype=torch.float32)[: self.dim // 2] / self.dim))
        self.register_buffer("theta", theta, persistent=False)
        self.build_rope_cache(self.max_seq_len)

    def build_rope_cache(self, max_seq_len: int) -> None:
        pos = torch.arange(max_seq_len, dtype=torch.float32, device=self.theta.device)
        ang = torch.outer(pos, self.theta)                                    # [max_seq, dim/2]
        self.register_buffer("cache", torch.stack([ang.cos(), ang.sin()], dim=-1), persistent=False)

    def _cos_sin(self, seq_len: int, input_pos: Optional[torch.Tensor]):
        cache = self.cache[:seq_len] if input_pos is None else self.cache[input_pos]
        if input_pos is None:
            cache = cache[None]                       # [1, s, d/2, 2]
        return cache[..., 0].unsqueeze(2), cache[..., 1].unsqueeze(2)          # [b|1, s, 1, d/2]


class RotaryPositionalEmbeddings(_RopeBase):
    def forward(self, x: torch.Tensor, input_pos: Optional[torch.Tensor] = None) -> torch.Tensor:
        """``x`` ``[b, s, n_heads, d]``; ``input_pos`` ``[b, s]`` (or ``None`` for ``0..s-1``)."""
        cos, sin = self._cos_sin(x.shape[1], input_pos)
        xf = x.float()
        x1, x2 = xf[..., : self.dim // 2], xf[..., self.dim // 2:]
        return torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin], dim=-1).to(x.dtype)


class LlamaRotaryPositionalEmbeddings(_RopeBase):
    def forward(self, x: torch.Tensor, input_pos: Optional[torch.Tensor] = None) -> torch.Tensor:
        cos, sin = self._cos_sin(x.shape[1], input_pos)
        xf = x.float().reshape(*x.shape[:-1], -1, 2)
        x1, x2 = xf[..., 0], xf[..., 1]
        out = torch.stack([x1 * cos - x2 * sin, x2 * cos + x1 * sin], dim=-1)
        return out.flatten(-2).to(x.dtype)
