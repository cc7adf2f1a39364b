"""RMSNorm with fp32 statistics; the parameter is named ``scale`` (``muse/layers/rms_norm.py:50-80``)."""
import torch
from torch import nn

from .. import ops


class RMSNorm(nn.Module):
    def __init__(self, dim: int, eps: float = 1e-6):
        super().__init__()
        self.dim, self.eps = dim, eps
        self.scale = nn.Parameter(torch.ones(dim))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        shape = x.shape
        if x.is_cuda and x.dtype == torch.bfloat16 and self.scale.dtype == torch.bfloat16:
            return ops.rms_norm(x.reshape(-1, shape[-1]), self.scale, self.eps).view(shape)
        xf = x.float()
        y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + self.eps)
        return (y * self.scale.float()).to(x.dtype)
