"""Generic pre-norm transformer blocks and decoder (``muse/layers/transformer.py:63-192,195-367,385-731``)."""
import copy
from typing import List, Optional, Union

import torch
from torch import nn

from .. import ops


class TransformerSelfAttentionLayer(nn.Module):
    """``h = x + sa_scale(attn(sa_norm(x)))``; ``out = h + mlp_scale(mlp(mlp_norm(h)))``."""

    def __init__(self, attn: nn.Module, mlp: nn.Module, sa_norm: Optional[nn.Module] = None,
                 mlp_norm: Optional[nn.Module] = None, sa_scale: Optional[nn.Module] = None,
                 mlp_scale: Optional[nn.Module] = None):
        super().__init__()
        self.attn, self.mlp = attn, mlp
        self.sa_norm = sa_norm or nn.Identity()
        self.mlp_norm = mlp_norm or nn.Identity()
        self.sa_scale = sa_scale or nn.Identity()
        self.mlp_scale = mlp_scale or nn.Identity()

    def setup_cache(self, batch_size: int, dtype: torch.dtype, max_seq_len: Optional[int] = None) -> None:
        self.attn.setup_cache(batch_size, dtype, max_seq_len)

    def reset_cache(self) -> None:
        self.attn.reset_cache()

    def forward(self, x: torch.Tensor, mask: Optional[torch.Tensor] = None, input_pos: Optional[torch.Tensor] = None,
                **kwargs) -> torch.Tensor:
        h = x + self.sa_scale(self.attn(self.sa_norm(x), mask=mask, input_pos=input_pos, **kwargs))
        return h + self.mlp_scale(self.mlp(self.mlp_norm(h)))


class TransformerCrossAttentionLayer(nn.Module):
    """Cross-attention block: queries from the decoder stream, keys/values from ``encoder_input``; skipped (identity)
    when no encoder input is given and nothing is cached."""

    def __init__(self, attn: nn.Module, mlp: nn.Module, ca_norm: Optional[nn.Module] = None,
                 mlp_norm: Optional[nn.Module] = None, ca_scale: Optional[nn.Module] = None,
                 mlp_scale: Optional[nn.Module] = None):
        super().__init__()
        if getattr(attn, "pos_embeddings", None) is not None:
            raise ValueError("cross-attention takes no positional embeddings")
        self.attn, self.mlp = attn, mlp
        self.ca_norm = ca_norm or nn.Identity()
        self.mlp_norm = mlp_norm or nn.Identity()
        self.ca_scale = ca_scale or nn.Identity()
        self.mlp_scale = mlp_scale or nn.Identity()

    def forward(self, x: torch.Tensor, encoder_input: Optional[torch.Tensor] = None,
                encoder_mask: Optional[torch.Tensor] = None, **kwargs) -> torch.Tensor:
        if encoder_input is None:
            return x
        h = x + self.ca_scale(self.attn(self.ca_norm(x), y=encoder_input, mask=encoder_mask))
        return h + self.mlp_scale(self.mlp(self.mlp_norm(h)))


def _clones(module: nn.Module, n: int) -> nn.ModuleList:
    return nn.ModuleList([copy.deepcopy(module) for _ in range(n)])


class TransformerDecoder(nn.Module):
    """Embedding -> layers -> norm -> output projection.

    ``layers`` is a list of blocks or one block to be repeated ``num_layers`` times.  ``skip_output_layer`` returns
    the normalised hidden states (the trainer's chunked loss applies the head itself, ``transformer.py:721-722``);
    ``output_hidden_states`` lists layer indices whose inputs are returned before the final output.
    """

    def __init__(self, tok_embeddings: nn.Embedding, layers: Union[nn.Module, List[nn.Module], nn.ModuleList],
                 max_seq_len: int, num_heads: int, head_dim: int, norm: nn.Module, output: nn.Module,
                 num_layers: Optional[int] = None, output_hidden_states: Optional[List[int]] = None):
        super().__init__()
        if isinstance(layers, nn.ModuleList):
            self.layers = layers
        elif isinstance(layers, list):
            self.layers = nn.ModuleList(layers)
        else:
            if num_layers is None:
                raise ValueError("num_layers is required when one layer is given")
            self.layers = _clones(layers, num_layers)
        self.tok_embeddings, self.norm, self.output = tok_embeddings, norm, output
        self.max_seq_len, self.num_heads, self.head_dim = max_seq_len, num_heads, head_dim
        self.output_hidden_states = output_hidden_states or []
        self.skip_output_layer = False

    def setup_caches(self, batch_size: int, dtype: torch.dtype, max_seq_len: Optional[int] = None) -> None:
        for layer in self.layers:
            if hasattr(layer, "setup_cache"):
                layer.setup_cache(batch_size, dtype, max_seq_len or self.max_seq_len)

    def caches_are_enabled(self) -> bool:
        return any(getattr(getattr(l, "attn", None), "cache_enabled", False) for l in self.layers)

    def reset_caches(self) -> None:
        if not self.caches_are_enabled():
            raise RuntimeError("KV caches are not set up; call setup_caches() first")
        for layer in self.layers:
            if hasattr(layer, "reset_cache"):
                layer.reset_cache()

    def forward(self, tokens: torch.Tensor, mask: Optional[torch.Tensor] = None,
                encoder_input: Optional[torch.Tensor] = None, encoder_mask: Optional[torch.Tensor] = None,
                input_pos: Optional[torch.Tensor] = None):
        if tokens.shape[1] > self.max_seq_len:
            raise ValueError(f"sequence length {tokens.shape[1]} exceeds max_seq_len {self.max_seq_len}")
        h = self.tok_embeddings(tokens)
        hidden = []
        for i, layer in enumerate(self.layers):
            if i in self.output_hidden_states:
                hidden.append(h)
            if isinstance(layer, TransformerCrossAttentionLayer):
                h = layer(h, encoder_input=encoder_input, encoder_mask=encoder_mask)
            else:
                h = layer(h, mask=mask, input_pos=input_pos)
        h = self.norm(h)
        if self.skip_output_layer:
            out = h
        else:
            shape = h.shape
            out = self.output(h) if not isinstance(self.output, nn.Linear) else ops.linear(
                h.reshape(-1, shape[-1]), self.output.weight, self.output.bias).view(*shape[:-1], -1)
        return out if not hidden else hidden + [out]
