"""SwiGLU feed-forward ``w2(silu(w1 x) * w3 x)`` (``muse/layers/feed_forward.py:44-83``)."""
import torch
from torch import nn

from .. import ops


class FeedForward(nn.Module):
    def __init__(self, dim: int, hidden_dim: int):
        super().__init__()
        self.w1 = nn.Linear(dim, hidden_dim, bias=False)
        self.w2 = nn.Linear(hidden_dim, dim, bias=False)
        self.w3 = nn.Linear(dim, hidden_dim, bias=False)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        shape = x.shape
        x2 = x.reshape(-1, shape[-1])
        gate_up = torch.cat([ops.linear(x2, self.w1.weight), ops.linear(x2, self.w3.weight)], dim=-1)
        return ops.linear(ops.swiglu(gate_up), self.w2.weight).view(shape)
