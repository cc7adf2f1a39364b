"""LayerNorm computed in fp32 whatever the input dtype (``muse/layers/layer_norm.py:40-62``)."""
import torch
from torch import nn
from torch.nn import functional as F


class Fp32LayerNorm(nn.LayerNorm):
    def forward(self, x: torch.Tensor) -> torch.Tensor:
        w = self.weight.float() if self.weight is not None else None
        b = self.bias.float() if self.bias is not None else None
        return F.layer_norm(x.float(), self.normalized_shape, w, b, self.eps).to(x.dtype)
