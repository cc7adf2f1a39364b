"""Activation checkpointing per decoder layer (``muse/training/activations.py:29-78``).

The reference wraps each layer class in torch's checkpoint wrapper from 32k context up.  Here a layer is wrapped so
that its forward runs under ``torch.utils.checkpoint`` (non-reentrant): only the layer's inputs stay alive and the
layer is recomputed in backward.  At 8k context the engine does not need it (activations of the whole 1.9B model
are ~15 GB on a 180 GB part); it exists for the 64k/128k stages and for parity of the CLI flag.

``mode="mlp"`` is the selective form for a 180 GB part: only the feed-forward block of each layer is recomputed
(gate/up projection and SwiGLU, the three widest tensors a layer keeps), attention and its projections are not.
Per token and layer of Qwen3-1.9B-KSA that keeps about 14k of 32k values, at the price of one extra gate/up GEMM
(about a seventh of a layer's forward arithmetic) instead of a whole extra forward pass.
"""
from __future__ import annotations

from typing import Iterable, Optional, Tuple

import torch
import torch.nn as nn
from torch.utils.checkpoint import checkpoint


class CheckpointedLayer(nn.Module):
    def __init__(self, layer: nn.Module):
        super().__init__()
        self._checkpoint_wrapped_module = layer

    def forward(self, x, delta, meta, collect=None):
        if not torch.is_grad_enabled() or collect is not None:
            return self._checkpoint_wrapped_module(x, delta, meta, collect)
        return checkpoint(self._checkpoint_wrapped_module, x, delta, meta, None, use_reentrant=False)

    def __getattr__(self, name):
        try:
            return super().__getattr__(name)
        except AttributeError:
            return getattr(self._modules["_checkpoint_wrapped_module"], name)


def set_activation_checkpointing(model: nn.Module, auto_wrap_policy: Optional[Tuple[type, ...]] = None,
                                 every: int = 1, mode: str = "full") -> int:
    """Checkpoint every ``every``-th layer of ``model.layers`` whose class is in ``auto_wrap_policy``; returns the
    count.  ``mode="full"`` recomputes the whole layer, ``mode="mlp"`` only its feed-forward block (layers that have
    a ``recompute_mlp`` switch)."""
    if mode not in ("full", "mlp"):
        raise ValueError(f"activation checkpointing mode must be 'full' or 'mlp', not {mode!r}")
    classes = tuple(auto_wrap_policy) if auto_wrap_policy else None
    layers = getattr(model, "layers", None)
    if layers is None:
        return 0
    n = 0
    for i, layer in enumerate(list(layers)):
        if isinstance(layer, CheckpointedLayer) or i % every:
            continue
        if classes is None or isinstance(layer, classes):
            if mode == "mlp":
                if not hasattr(layer, "recompute_mlp"):
                    continue
                layer.recompute_mlp = True
            else:
                layers[i] = CheckpointedLayer(layer)
            n += 1
    return n
