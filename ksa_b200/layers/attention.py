"""Generic grouped-query multi-head attention block (``muse/layers/attention.py:21-321``).

Order of operations as in the reference's generic block: projections -> RoPE -> optional q/k norms -> attention ->
output projection (the Qwen3 models apply QK-norm *before* RoPE and use their own fused block).  A ``KVCache`` can be
attached for incremental decoding; ``y`` switches the block to cross-attention.
"""
from typing import Optional

import torch
from torch import nn

from .. import ops
from .attention_utils import get_attention_backend
from .kv_cache import KVCache


def _proj(x: torch.Tensor, lin: nn.Linear) -> torch.Tensor:
    shape = x.shape
    y = ops.linear(x.reshape(-1, shape[-1]), lin.weight, lin.bias)
    return y.view(*shape[:-1], -1)


class MultiHeadAttention(nn.Module):
    def __init__(self, embed_dim: int, num_heads: int, num_kv_heads: int, head_dim: int,
                 pos_embeddings: Optional[nn.Module] = None, q_norm: Optional[nn.Module] = None,
                 k_norm: Optional[nn.Module] = None, kv_cache: Optional[KVCache] = None, max_seq_len: int = 4096,
                 is_causal: bool = True, attn_dropout: float = 0.0, bias: bool = False,
                 attention_backend: str = "tensor_core", sliding_window: int = -1):
        super().__init__()
        if num_heads % num_kv_heads:
            raise ValueError(f"num_heads ({num_heads}) must be a multiple of num_kv_heads ({num_kv_heads})")
        if (q_norm is None) != (k_norm is None):
            raise ValueError("q_norm and k_norm must be set together")
        if attn_dropout:
            raise ValueError("attention dropout is not supported by the attention kernels")
        self.embed_dim, self.num_heads, self.num_kv_heads, self.head_dim = embed_dim, num_heads, num_kv_heads, head_dim
        self.max_seq_len, self.is_causal, self.sliding_window = max_seq_len, is_causal, sliding_window
        self.q_proj = nn.Linear(embed_dim, num_heads * head_dim, bias=bias)
        self.k_proj = nn.Linear(embed_dim, num_kv_heads * head_dim, bias=bias)
        self.v_proj = nn.Linear(embed_dim, num_kv_heads * head_dim, bias=bias)
        self.output_proj = nn.Linear(num_heads * head_dim, embed_dim, bias=bias)
        self.pos_embeddings, self.q_norm, self.k_norm = pos_embeddings, q_norm, k_norm
        self.kv_cache = kv_cache
        self.cache_enabled = kv_cache is not None
        self.attn = get_attention_backend(attention_backend)

    def setup_cache(self, batch_size: int, dtype: torch.dtype, max_seq_len: Optional[int] = None) -> None:
        self.kv_cache = KVCache(batch_size, max_seq_len or self.max_seq_len, self.num_kv_heads, self.head_dim, dtype)
        self.kv_cache.to(self.q_proj.weight.device)
        self.cache_enabled = True

    def reset_cache(self) -> None:
        if self.kv_cache is None:
            raise RuntimeError("no KV cache has been set up")
        self.kv_cache.reset()

    def forward(self, x: torch.Tensor, y: Optional[torch.Tensor] = None, mask: Optional[torch.Tensor] = None,
                input_pos: Optional[torch.Tensor] = None, cu_seqlens: Optional[torch.Tensor] = None) -> torch.Tensor:
        """``x`` ``[b, s, d]`` queries; ``y`` ``[b, s_y, d]`` the key/value source (``None`` = self-attention)."""
        b, s, _ = x.shape
        src = x if y is None else y
        q = _proj(x, self.q_proj).view(b, s, self.num_heads, self.head_dim)
        k = _proj(src, self.k_proj).view(b, src.shape[1], self.num_kv_heads, self.head_dim)
        v = _proj(src, self.v_proj).view(b, src.shape[1], self.num_kv_heads, self.head_dim)
        if self.pos_embeddings is not None:
            q = self.pos_embeddings(q, input_pos=input_pos)
            if y is None:
                k = self.pos_embeddings(k, input_pos=input_pos)
        if self.q_norm is not None:
            q, k = self.q_norm(q), self.k_norm(k)
        if self.cache_enabled and self.kv_cache is not None and y is None:
            k, v = self.kv_cache.update(k, v)
        causal = self.is_causal and y is None
        out = self.attn(q, k, v, mask=mask, is_causal=causal, window=self.sliding_window, cu_seqlens=cu_seqlens)
        return _proj(out.reshape(b, s, self.num_heads * self.head_dim), self.output_proj)
