"""DCP directory -> a single ``torch.save`` file or sharded safetensors, no key remapping
(``muse/tools/dcp2torch.py:21-148``)."""
from __future__ import annotations

import argparse
from pathlib import Path

import torch

from ..models.base import save_sharded_safetensors
from ..training.checkpoint import dcp_to_state_dict
from .convert import flatten_model_state


def convert(dcp_dir: str, out: str, model_only: bool = True, use_safetensor: bool = False, dtype=None) -> str:
    sd = dcp_to_state_dict(dcp_dir)
    state = flatten_model_state(sd) if model_only else sd
    if dtype is not None and model_only:
        state = {k: v.to(dtype) for k, v in state.items()}
    out_path = Path(out)
    if use_safetensor or str(out_path).endswith(".safetensors") or out_path.suffix == "":
        save_sharded_safetensors(state, str(out_path if out_path.suffix == "" else out_path.parent))
    else:
        out_path.parent.mkdir(parents=True, exist_ok=True)
        torch.save(state, str(out_path))
    return str(out_path)


def main(argv=None) -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("dcp_dir")
    ap.add_argument("out")
    ap.add_argument("--all", action="store_true", help="keep optimizer and training state too (torch.save only)")
    ap.add_argument("--safetensors", action="store_true")
    a = ap.parse_args(argv)
    print(convert(a.dcp_dir, a.out, model_only=not a.all, use_safetensor=a.safetensors))


if __name__ == "__main__":
    main()
