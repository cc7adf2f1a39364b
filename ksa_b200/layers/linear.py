"""Output projection that shares another module's weight (``muse/layers/linear.py:58-93``)."""
import torch
from torch import nn

from .. import ops


class TiedLinear(nn.Module):
    """``x @ tied.weight.T``: holds a reference to the owning module, never a copy, so FSDP-style flat storage and
    checkpoint loading keep one tensor."""

    def __init__(self, tied_module: nn.Module):
        super().__init__()
        object.__setattr__(self, "_tied", tied_module)     # not registered: the weight has one owner
        if not hasattr(tied_module, "weight"):
            raise AttributeError("the tied module has no weight")

    @property
    def weight(self) -> torch.Tensor:
        return self._tied.weight

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        shape = x.shape
        y = ops.linear(x.reshape(-1, shape[-1]), self.weight)
        return y.view(*shape[:-1], -1)
