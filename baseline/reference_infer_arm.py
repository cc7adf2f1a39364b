"""Reference arm of ``ksa_b200.tools.infer_bench``: the reference's own HF ``trust_remote_code`` template
(``examples/pretrain/hf_template`` of the reference tree, copied unmodified into a scratch directory) with random
weights of the KSA-4B shape, timed through its public API: ``AutoModelForCausalLM`` + ``generate``
(``examples/inference/inference.py:20-82``), batch 1, one GPU, greedy.

The template cannot express a stack with real full-attention layers (it builds a layer only when
``use_summary_attention`` and the layer's ``summary_layer_freq`` entry agree, ``modeling_qwen3sa.py:889-895``), so the
"full" quarter is what the reference itself ships: summary layers with a 1024-chunk window
(``summary_sliding_chunk_num = "([8]*3+[1024]*1)*9"``).  Batch sizes above one and tensor parallelism do not exist in
the reference; asking for them prints the ``unavailable`` line.  Any exception while importing or running the template
(for instance a ``transformers`` release it was not written for) is reported the same way, with its text.
"""
from __future__ import annotations

import json
import os
import shutil
import sys
import tempfile
import traceback

HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.path.join(HERE, "_ref")
TEMPLATE = os.path.join(REF, "hf_template")     # copied there from the reference tree when the reference is installed

KSA_4B = {"hidden_size": 2560, "intermediate_size": 9728, "num_hidden_layers": 36, "num_attention_heads": 32,
          "num_key_value_heads": 8, "head_dim": 128, "vocab_size": 151936, "summary_token_begin": 151936,
          "summary_chunk_size": 128, "summary_token_num": 1, "summary_sliding_chunk_num": "([8]*3+[1024]*1)*9",
          "tie_word_embeddings": False, "rope_theta": 1000000, "max_position_embeddings": 131072 + 4096}


def _unavailable(why: str) -> dict:
    return {"impl": "reference", "unavailable": " ".join(str(why).split())[:400]}


def run_reference_infer_arm(prompt_len: int, decode: int, batch: int, world: int, template_dir: str = None) -> dict:
    if batch != 1:
        return _unavailable("the reference's HF attention raises for batch != 1 "
                            "(examples/pretrain/hf_template/modeling_qwen3sa.py:753-754)")
    if world != 1:
        return _unavailable("the reference has no tensor parallelism (single-device inference only)")
    src = template_dir or TEMPLATE
    if not os.path.isdir(src):
        root = os.environ.get("KSA_REFERENCE_ROOT", "")      # a checkout of the reference, when it is not installed
        src = os.path.join(root, "examples", "pretrain", "hf_template") if root else src
    if not os.path.isdir(src):
        return _unavailable(f"the reference's HF template is not on this machine ({TEMPLATE})")
    work = tempfile.mkdtemp(prefix="ref_hf_")
    try:
        return _run(src, work, prompt_len, decode)
    except BaseException as e:  # noqa: BLE001 - import errors of the template surface as all kinds of exceptions
        tb = traceback.format_exc().strip().splitlines()
        where = next((l.strip() for l in reversed(tb) if "modeling_qwen3sa.py" in l), "")
        return _unavailable(f"{type(e).__name__}: {e} [{where}] (reference template with transformers "
                            f"{_transformers_version()}; it pins transformers >= 4.57 of the 4.x line)")
    finally:
        shutil.rmtree(work, ignore_errors=True)


def _transformers_version() -> str:
    try:
        import transformers
        return transformers.__version__
    except Exception:  # noqa: BLE001
        return "?"


def _run(src: str, work: str, prompt_len: int, decode: int) -> dict:
    import torch
    sys.path.insert(0, REF)              # summary_attn and flash_attn.cute of the reference's wheels
    try:
        import flash_attn
        flash_attn.__path__.append(os.path.join(REF, "flash_attn"))
    except Exception:  # noqa: BLE001
        pass
    for name in os.listdir(src):
        if name.endswith((".py", ".json")):
            shutil.copy(os.path.join(src, name), os.path.join(work, name))
    cfg_path = os.path.join(work, "config.json")
    cfg = json.load(open(cfg_path))
    cfg.update(KSA_4B)
    json.dump(cfg, open(cfg_path, "w"))
    from transformers import AutoConfig, AutoModelForCausalLM
    config = AutoConfig.from_pretrained(work, trust_remote_code=True)
    torch.manual_seed(0)
    with torch.device("cuda"):
        model = AutoModelForCausalLM.from_config(config, trust_remote_code=True, torch_dtype=torch.bfloat16)
    model = model.to(torch.bfloat16).eval()
    g = torch.Generator().manual_seed(1)
    prompt = torch.randint(0, 150000, (1, prompt_len), generator=g).cuda()

    def timed(new_tokens: int) -> float:
        torch.cuda.synchronize()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        with torch.no_grad():
            model.generate(prompt, max_new_tokens=new_tokens, do_sample=False, eos_token_id=None, pad_token_id=0)
        e.record()
        torch.cuda.synchronize()
        return s.elapsed_time(e)

    timed(2)                                   # warm-up (JIT compilation of the summary-attention back end)
    ms_prefill = timed(1)
    ms_total = timed(1 + decode)
    ms_decode = max(ms_total - ms_prefill, 0.0)
    return {"impl": "reference", "model": "ksa-4b shape, reference HF template", "tp": 1, "batch": 1,
            "prompt_len": prompt_len, "decode_steps": decode, "dtype": "bf16",
            "prefill_ms": ms_prefill, "prefill_tokens_per_s": prompt_len / (ms_prefill / 1e3),
            "decode_ms_per_step": ms_decode / max(decode, 1), "decode_tokens_per_s": decode / (ms_decode / 1e3) if ms_decode else None,
            "transformers": _transformers_version(), "data": "uniform random prompt, random-init weights"}
