"""DCP checkpoint -> HuggingFace directory (sharded safetensors + index + template files).

Same job and CLI as ``examples/pretrain/convert/convert.py:55-101`` and ``convert/checkpoint.py:114-223`` of the
reference: read the DCP directory in ONE process without a process group, take ``app.model``, optionally remap the
reference's parameter names to HF names (the summary embedding is appended to ``embed_tokens`` and ``lm_head`` is
zero-padded to the same vocabulary), cast, shard at 4 GB into ``model-0000i-of-0000n.safetensors`` +
``model.safetensors.index.json``, copy the template's ``*.json / *.py / *.txt`` and patch ``vocab_size`` in
``config.json`` to the checkpoint's embedding rows.

    python -m ksa_b200.tools.convert --dcp_path OUT --step global_step5000 --base_model_path ksa_b200/hf --remap muse2hf
"""
from __future__ import annotations

import argparse
import json
import os
import shutil
from typing import Dict, Optional

import torch

from ..models.base import save_sharded_safetensors
from ..models.qwen3_ksa import Qwen3Model
from ..training.checkpoint import dcp_to_state_dict

_DTYPES = {"bf16": torch.bfloat16, "fp16": torch.float16, "fp32": torch.float32}


def flatten_model_state(sd: dict) -> Dict[str, torch.Tensor]:
    """``app.model.<name>`` entries of a loaded DCP tree (nested or flat) as ``{name: tensor}``."""
    node = sd
    for key in ("app", "model"):
        if isinstance(node, dict) and key in node:
            node = node[key]
    out: Dict[str, torch.Tensor] = {}

    def walk(prefix: str, n) -> None:
        if torch.is_tensor(n):
            out[prefix] = n
        elif isinstance(n, dict):
            for k, v in n.items():
                walk(f"{prefix}.{k}" if prefix else str(k), v)
    walk("", node)
    if any(k.startswith("app.model.") for k in out):
        out = {k[len("app.model."):]: v for k, v in out.items() if k.startswith("app.model.")}
    return out


def dcp_to_safetensors(dcp_dir: str, out_dir: str, dtype: str = "bf16", remap: str = "none",
                       max_gb_per_shard: float = 4.0) -> dict:
    state = flatten_model_state(dcp_to_state_dict(dcp_dir))
    if not state:
        raise RuntimeError(f"{dcp_dir}: no app.model.* tensors found")
    if remap == "muse2hf":
        state = Qwen3Model.muse_to_hf_keys(state)
    elif remap != "none":
        raise ValueError(f"unknown remap {remap!r}")
    td = _DTYPES[dtype]
    state = {k: v.to(td).contiguous() for k, v in state.items()}
    return save_sharded_safetensors(state, out_dir, f"{int(max_gb_per_shard * 1024)}MB")


def sync_vocab_size(hf_dir: str) -> Optional[int]:
    """Set ``vocab_size`` in config.json to the rows of ``embed_tokens`` actually stored."""
    from safetensors import safe_open
    cfg_path = os.path.join(hf_dir, "config.json")
    if not os.path.exists(cfg_path):
        return None
    rows = None
    for f in sorted(os.listdir(hf_dir)):
        if f.endswith(".safetensors"):
            with safe_open(os.path.join(hf_dir, f), "pt") as sf:
                for k in sf.keys():
                    if k.endswith("embed_tokens.weight") or k.endswith("tok_embeddings.weight"):
                        rows = sf.get_slice(k).get_shape()[0]
    if rows is None:
        return None
    cfg = json.load(open(cfg_path))
    cfg["vocab_size"] = int(rows)
    json.dump(cfg, open(cfg_path, "w"), indent=2)
    return rows


def convert_dcp_to_hf(checkpoint_dir: str, model_path: str, base_model_path: str, dtype: str = "bf16",
                      output_subdir: str = "hf", remap: str = "none", config_overrides: Optional[dict] = None) -> str:
    real = os.path.join(checkpoint_dir, model_path)
    out = os.path.join(real, output_subdir)
    dcp_to_safetensors(real, out, dtype=dtype, remap=remap)
    for f in os.listdir(base_model_path):
        if f == "model.safetensors.index.json":
            continue
        if f.endswith((".json", ".py", ".txt")):
            shutil.copy(os.path.join(base_model_path, f), os.path.join(out, f))
    if config_overrides:
        p = os.path.join(out, "config.json")
        cfg = json.load(open(p))
        cfg.update(config_overrides)
        json.dump(cfg, open(p, "w"), indent=2)
    sync_vocab_size(out)
    return out


def hf_config_from_model_config(cfg) -> dict:
    """HF ``config.json`` fields for a framework model config (merged into the template's config)."""
    out = {
        "hidden_size": cfg.embed_dim, "intermediate_size": cfg.intermediate_dim, "num_hidden_layers": cfg.num_layers,
        "num_attention_heads": cfg.num_heads, "num_key_value_heads": cfg.num_kv_heads, "head_dim": cfg.head_dim,
        "rms_norm_eps": cfg.norm_eps, "rope_theta": cfg.rope_base, "max_position_embeddings": cfg.max_seq_len,
        "tie_word_embeddings": cfg.tie_word_embeddings, "vocab_size": cfg.vocab_size,
    }
    if getattr(cfg, "summary_enabled", False):
        out.update({
            "use_summary_attention": True, "summary_chunk_size": cfg.summary_chunk_size,
            "summary_token_num": cfg.summary_token_num, "summary_token_begin": cfg.summary_token_begin,
            "summary_sliding_chunk_num": cfg.summary_sliding_chunk_num,
            "summary_layer_freq": [int(b) for b in cfg.get_layer_is_summary()],
            "summary_chunk_position_ids_type": cfg.summary_chunk_position_ids_type,
            "summary_token_position_ids_type": cfg.summary_token_position_ids_type,
            "summary_independent_parameters": cfg.summary_independent_parameters,
            "summary_independent_attention_layernorm": cfg.summary_independent_attention_layernorm,
            "summary_independent_qk_norm": cfg.summary_independent_qk_norm,
        })
    return out


def model_config_from_hf_config(hf: dict):
    """The framework model config for an HF ``config.json`` written by ``hf_config_from_model_config`` (its inverse).

    With independent summary parameters the HF embedding holds the summary-token rows after the text vocabulary
    (``sync_vocab_size`` records that row count), so the text vocabulary ends where the summary tokens begin."""
    from ..config.model_config import Qwen3Config, Qwen3SummaryAttentionConfig
    common = dict(
        vocab_size=hf["vocab_size"], embed_dim=hf["hidden_size"], intermediate_dim=hf["intermediate_size"],
        num_layers=hf["num_hidden_layers"], num_heads=hf["num_attention_heads"],
        num_kv_heads=hf.get("num_key_value_heads", hf["num_attention_heads"]),
        head_dim=hf.get("head_dim", hf["hidden_size"] // hf["num_attention_heads"]),
        norm_eps=hf.get("rms_norm_eps", 1e-6), rope_base=hf.get("rope_theta", 10000.0),
        max_seq_len=hf.get("max_position_embeddings", 131072), tie_word_embeddings=hf.get("tie_word_embeddings", False),
        q_norm=True, k_norm=True, rope_impl="hf")
    if hf.get("eos_token_id") is not None:
        common["eos_token_id"] = hf["eos_token_id"]
    if not hf.get("use_summary_attention", False):
        return Qwen3Config(**common)
    n_sum, begin = hf.get("summary_token_num", 1), hf.get("summary_token_begin")
    independent = hf.get("summary_independent_parameters", False)
    if independent and begin is not None and begin + n_sum == hf["vocab_size"]:
        common["vocab_size"] = begin
    return Qwen3SummaryAttentionConfig(
        use_summary_attention=True, summary_chunk_size=hf["summary_chunk_size"], summary_token_num=n_sum,
        summary_token_begin=begin if begin is not None else common["vocab_size"],
        summary_sliding_chunk_num=hf["summary_sliding_chunk_num"], summary_layer_freq=hf["summary_layer_freq"],
        summary_chunk_position_ids_type=hf.get("summary_chunk_position_ids_type", "origin"),
        summary_token_position_ids_type=hf.get("summary_token_position_ids_type", "last_chunk_slice_right"),
        summary_independent_parameters=independent,
        summary_independent_attention_layernorm=hf.get("summary_independent_attention_layernorm", False),
        summary_independent_qk_norm=hf.get("summary_independent_qk_norm", False), **common)


def load_hf_checkpoint(model_dir: str, device: str = "cpu", dtype=None):
    """Build this package's model (for ``KsaInferenceEngine``) from a converted checkpoint directory: the architecture
    from its ``config.json``, the weights from its safetensors under the Hugging Face parameter names."""
    from ..models import get_model_class
    cfg = model_config_from_hf_config(json.load(open(os.path.join(model_dir, "config.json"))))
    return get_model_class(cfg.model_class).from_pretrained(model_dir, config=cfg, device=device, dtype=dtype)


def main(argv=None) -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--dcp_path", required=True, help="training output dir containing global_step* subdirs")
    ap.add_argument("--step", required=True, help="e.g. global_step5000")
    ap.add_argument("--base_model_path", required=True, help="HF template dir (tokenizer/config/modeling files)")
    ap.add_argument("--dtype", default="bf16", choices=sorted(_DTYPES))
    ap.add_argument("--remap", default="none", choices=["none", "muse2hf"])
    args = ap.parse_args(argv)
    print(convert_dcp_to_hf(args.dcp_path, args.step, args.base_model_path, args.dtype, remap=args.remap))


if __name__ == "__main__":
    main()
