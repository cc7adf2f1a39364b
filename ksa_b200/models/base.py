"""Model registry and base class.

Mirrors the reference's registry (``muse/models/__init__.py:12-76``) and ``Model`` base
(``muse/models/base.py:19-412``): name -> class lookup, HF-directory load/save with sharded
safetensors + index, initializer lookup, optimizer parameter groups, and the hooks the trainer needs
(`get_layers_to_shard`, `get_checkpointable_module_classes`, Muse<->HF key conversion).
"""
from __future__ import annotations

import json
import os
import re
from pathlib import Path
from typing import Callable, Dict, Iterable, List, Optional, Tuple, Type

import torch
import torch.nn as nn

_MODEL_REGISTRY: Dict[str, Type["Model"]] = {}


def register_model(name: Optional[str] = None):
    def deco(cls):
        _MODEL_REGISTRY[name or cls.__name__] = cls
        return cls
    return deco


def get_model_class(name: str) -> Type["Model"]:
    if name not in _MODEL_REGISTRY:
        raise KeyError(f"unknown model {name!r}; registered: {sorted(_MODEL_REGISTRY)}")
    return _MODEL_REGISTRY[name]


def list_models() -> List[str]:
    return sorted(_MODEL_REGISTRY)


def parse_size(text: str) -> int:
    m = re.fullmatch(r"\s*(\d+(?:\.\d+)?)\s*([KMGT]?)B?\s*", str(text), re.I)
    if not m:
        raise ValueError(f"cannot parse size {text!r}")
    mult = {"": 1, "K": 1 << 10, "M": 1 << 20, "G": 1 << 30, "T": 1 << 40}[m.group(2).upper()]
    return int(float(m.group(1)) * mult)


def shard_state_dict(state: Dict[str, torch.Tensor], max_shard_bytes: int) -> List[Dict[str, torch.Tensor]]:
    """Greedy split of a state dict into shards of at most ``max_shard_bytes`` (a larger tensor gets its own)."""
    shards: List[Dict[str, torch.Tensor]] = [{}]
    size = 0
    for k, t in state.items():
        nbytes = t.numel() * t.element_size()
        if shards[-1] and size + nbytes > max_shard_bytes:
            shards.append({})
            size = 0
        shards[-1][k] = t
        size += nbytes
    return shards


def save_sharded_safetensors(state: Dict[str, torch.Tensor], out_dir: str, max_shard_size: str = "5GB",
                             metadata: Optional[dict] = None) -> dict:
    """Write ``model-0000i-of-0000n.safetensors`` (+ ``model.safetensors.index.json`` when n > 1)."""
    from safetensors.torch import save_file
    out = Path(out_dir)
    out.mkdir(parents=True, exist_ok=True)
    state = {k: v.detach().to("cpu").contiguous() for k, v in state.items()}
    shards = shard_state_dict(state, parse_size(max_shard_size))
    n = len(shards)
    weight_map = {}
    total = 0
    for i, shard in enumerate(shards, 1):
        name = "model.safetensors" if n == 1 else f"model-{i:05d}-of-{n:05d}.safetensors"
        save_file(shard, str(out / name), metadata={"format": "pt"})
        for k, t in shard.items():
            weight_map[k] = name
            total += t.numel() * t.element_size()
    index = {"metadata": {"total_size": total, **(metadata or {})}, "weight_map": weight_map}
    if n > 1:
        (out / "model.safetensors.index.json").write_text(json.dumps(index, indent=2))
    return index


def save_sharded_bin(state: Dict[str, torch.Tensor], out_dir: str, max_shard_size: str = "5GB") -> dict:
    """The ``torch.save`` form of the same layout: ``pytorch_model.bin``, or ``pytorch_model-0000i-of-0000n.bin`` +
    ``pytorch_model.bin.index.json`` (``muse/models/base.py:253-306``)."""
    out = Path(out_dir)
    out.mkdir(parents=True, exist_ok=True)
    state = {k: v.detach().to("cpu").contiguous() for k, v in state.items()}
    shards = shard_state_dict(state, parse_size(max_shard_size))
    n = len(shards)
    weight_map, total = {}, 0
    for i, shard in enumerate(shards, 1):
        name = "pytorch_model.bin" if n == 1 else f"pytorch_model-{i:05d}-of-{n:05d}.bin"
        torch.save(shard, str(out / name))
        for k, t in shard.items():
            weight_map[k] = name
            total += t.numel() * t.element_size()
    index = {"metadata": {"total_size": total}, "weight_map": weight_map}
    if n > 1:
        (out / "pytorch_model.bin.index.json").write_text(json.dumps(index, indent=2))
    return index


def load_hf_state_dict(model_dir: str, device: str = "cpu") -> Dict[str, torch.Tensor]:
    """Read every ``*.safetensors`` (or ``pytorch_model*.bin``) of an HF directory into one dict."""
    d = Path(model_dir)
    out: Dict[str, torch.Tensor] = {}
    st = sorted(d.glob("*.safetensors"))
    if st:
        from safetensors.torch import load_file
        for f in st:
            out.update(load_file(str(f), device=device))
        return out
    bins = sorted(d.glob("pytorch_model*.bin"))
    if not bins:
        raise FileNotFoundError(f"no *.safetensors or pytorch_model*.bin under {model_dir}")
    for f in bins:
        out.update(torch.load(str(f), map_location=device, weights_only=True))
    return out


def load_full_state_dict(model: nn.Module, state: Dict[str, torch.Tensor], allow_random_init_params=None,
                         skip_load_params=None, verbose: Optional[Callable[[str], None]] = None) -> Dict[str, List[str]]:
    """Load a whole-model state dict into an initialised model with the reference's rules
    (``muse/training/distributed.py:290-420``):

    * a parameter named in ``allow_random_init_params`` (exact names; a list or a comma-separated string) may be
      missing from ``state`` or have another shape there: it keeps its random initialisation;
    * a parameter whose name contains one of ``skip_load_params`` (substrings) is never loaded, even if present;
    * any other missing parameter, any other shape mismatch and any key of ``state`` the model does not have is an error.

    The model must already hold its initial values (``init_weights``).  Returns the names that kept them, by reason.
    """
    def as_list(v):
        if v is None:
            return []
        if isinstance(v, str):
            return [p.strip() for p in v.split(",") if p.strip()]
        return list(v)
    allow, skip = set(as_list(allow_random_init_params)), as_list(skip_load_params)
    own = model.state_dict()
    unexpected = sorted(set(state) - set(own))
    if unexpected:
        raise RuntimeError(f"the state dict holds {len(unexpected)} keys the model does not have: {unexpected[:5]}")
    kept: Dict[str, List[str]] = {"skipped": [], "missing": [], "shape": []}
    problems, to_load = [], {}
    for k, target in own.items():
        if any(p in k for p in skip):
            kept["skipped"].append(k)
        elif k not in state:
            (kept["missing"] if k in allow else problems).append(k)
        elif tuple(state[k].shape) != tuple(target.shape):
            if k in allow:
                kept["shape"].append(k)
            else:
                problems.append(f"{k}: model {tuple(target.shape)} vs state dict {tuple(state[k].shape)}")
        else:
            to_load[k] = state[k]
    if problems:
        raise RuntimeError("parameters missing from the state dict or of another shape; name them in "
                           f"allow_random_init_params or skip_load_params to keep their initialisation: {problems[:8]}")
    model.load_state_dict(to_load, strict=False)
    if verbose is not None:
        for reason, names in kept.items():
            for k in names:
                verbose(f"[load] {k}: kept its random initialisation ({reason})")
    return kept


class Model(nn.Module):
    """Base of every trainable model of the framework."""

    config_class = None

    def __init__(self, config):
        super().__init__()
        self.config = config

    # ---- trainer hooks -----------------------------------------------------------------
    def get_layers_to_shard(self) -> List[nn.Module]:
        """Modules that form one FSDP unit each (the root takes what is left)."""
        return list(getattr(self, "layers", []))

    def get_checkpointable_module_classes(self) -> Tuple[type, ...]:
        return tuple({type(m) for m in self.get_layers_to_shard()})

    def get_optimizer_grouped_parameters(self, weight_decay: float, learning_rate: Optional[float] = None) -> List[dict]:
        """One group, weight decay on every parameter, the learning rate when given (``muse/models/base.py:369-388``)."""
        group = {"params": [p for p in self.parameters() if p.requires_grad], "weight_decay": weight_decay}
        if learning_rate is not None:
            group["lr"] = learning_rate
        return [group]

    def get_hf_state_dict(self, state: Optional[Dict[str, torch.Tensor]] = None) -> Dict[str, torch.Tensor]:
        """The state dict under the Hugging Face parameter names (``muse/models/base.py:404-407``)."""
        return self.revert_hf_state_dict(state if state is not None else dict(self.state_dict()))

    def get_initializer(self) -> Callable[[nn.Module], None]:
        std = 0.02

        def init(module: nn.Module) -> None:
            for p in module.parameters(recurse=False):
                if p.dim() >= 2:
                    nn.init.normal_(p, 0.0, std)
                else:
                    nn.init.ones_(p)
        return init

    def init_weights(self, seed: Optional[int] = None) -> None:
        if seed is not None:
            torch.manual_seed(seed)
        init = self.get_initializer()
        with torch.no_grad():
            for m in self.modules():
                init(m)

    # ---- key conversion (identity unless a model overrides) --------------------------
    def convert_hf_state_dict(self, hf_state: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
        return hf_state

    def revert_hf_state_dict(self, state: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
        return state

    # ---- HF directory IO ------------------------------------------------------------
    @classmethod
    def from_pretrained(cls, model_dir: str, config=None, device: str = "cpu", dtype=None, strict: bool = True):
        from ..config import load_config
        if config is None:
            cfg_path = Path(model_dir) / "muse_config.json"
            if not cfg_path.exists():
                raise FileNotFoundError(f"{cfg_path} not found; pass config= explicitly")
            config = load_config(str(cfg_path))
        model = cls(config)
        state = model.convert_hf_state_dict(load_hf_state_dict(model_dir))
        missing, unexpected = model.load_state_dict(state, strict=False)
        if strict and (missing or unexpected):
            raise RuntimeError(f"state dict mismatch: missing {missing[:5]}..., unexpected {unexpected[:5]}...")
        if dtype is not None:
            model = model.to(dtype)
        return model.to(device)

    def save_pretrained(self, out_dir: str, max_shard_size: str = "5GB", dtype=None,
                        save_safetensors: bool = True) -> None:
        """HF-layout directory: weights under the Hugging Face names in shards of ``max_shard_size`` (safetensors, or
        ``torch.save`` files with ``save_safetensors=False``, ``muse/models/base.py:151-196``) plus the model config."""
        state = self.revert_hf_state_dict({k: v for k, v in self.state_dict().items()})
        if dtype is not None:
            state = {k: v.to(dtype) for k, v in state.items()}
        (save_sharded_safetensors if save_safetensors else save_sharded_bin)(state, out_dir, max_shard_size)
        self.config.save(os.path.join(out_dir, "muse_config.json"))

    def num_parameters(self) -> int:
        return sum(p.numel() for p in self.parameters())
