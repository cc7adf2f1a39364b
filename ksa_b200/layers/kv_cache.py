"""Append-only key/value cache ``[b, max_seq, n_kv, d]`` (``muse/layers/kv_cache.py:49-129``)."""
from typing import Tuple

import torch
from torch import nn


class KVCache(nn.Module):
    def __init__(self, batch_size: int, max_seq_len: int, num_kv_heads: int, head_dim: int, dtype=torch.bfloat16):
        super().__init__()
        shape = (batch_size, max_seq_len, num_kv_heads, head_dim)
        self.register_buffer("k_cache", torch.zeros(shape, dtype=dtype), persistent=False)
        self.register_buffer("v_cache", torch.zeros(shape, dtype=dtype), persistent=False)
        self.size = 0
        self.max_seq_len = max_seq_len

    def reset(self) -> None:
        self.k_cache.zero_()
        self.v_cache.zero_()
        self.size = 0

    def update(self, k: torch.Tensor, v: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        """Append ``[b, s, n_kv, d]`` and return views of everything cached so far."""
        b, s = k.shape[:2]
        if b > self.k_cache.shape[0]:
            raise ValueError(f"batch {b} exceeds the cache batch {self.k_cache.shape[0]}")
        if self.size + s > self.max_seq_len:
            raise ValueError(f"cache overflow: {self.size} + {s} > {self.max_seq_len}")
        self.k_cache[:b, self.size:self.size + s] = k
        self.v_cache[:b, self.size:self.size + s] = v
        self.size += s
        return self.k_cache[:b, :self.size], self.v_cache[:b, :self.size]
