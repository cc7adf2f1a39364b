#!/usr/bin/env python
"""Load a converted checkpoint and generate (counterpart of ``examples/inference/inference.py`` of the reference):
prints the completion and tokens/s.  By default the checkpoint's ``trust_remote_code`` model runs under
``transformers`` ``generate``, as in the reference; ``--engine`` runs this package's inference engine instead
(ring-buffer KV cache, sm_100a kernels and CUDA-graph decode on a GPU)."""
import argparse
import time

import torch
from transformers import AutoModelForCausalLM


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model_path", required=True)
    ap.add_argument("--prompt", default="Summarise the idea of summary attention in one sentence.")
    ap.add_argument("--prompt-ids", default=None, help="comma separated token ids (use when no tokenizer files exist)")
    ap.add_argument("--max-new-tokens", type=int, default=128)
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    ap.add_argument("--temperature", type=float, default=0.7)
    ap.add_argument("--top-p", type=float, default=0.9)
    ap.add_argument("--greedy", action="store_true")
    ap.add_argument("--engine", action="store_true", help="generate with ksa_b200's inference engine instead of HF generate")
    a = ap.parse_args()
    dtype = torch.bfloat16 if a.device.startswith("cuda") else torch.float32
    if a.engine:
        import os
        import sys
        sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))   # repository root
        from ksa_b200.tools.convert import load_hf_checkpoint
        model = load_hf_checkpoint(a.model_path, device=a.device, dtype=dtype).eval()
    else:
        model = AutoModelForCausalLM.from_pretrained(a.model_path, trust_remote_code=True, torch_dtype=dtype).to(a.device).eval()
    tok = None
    if a.prompt_ids:
        ids = torch.tensor([[int(t) for t in a.prompt_ids.split(",")]], device=a.device)
    else:
        from transformers import AutoTokenizer
        tok = AutoTokenizer.from_pretrained(a.model_path, trust_remote_code=True)
        text = a.prompt
        if getattr(tok, "chat_template", None):
            text = tok.apply_chat_template([{"role": "user", "content": a.prompt}], tokenize=False, add_generation_prompt=True)
        ids = tok(text, return_tensors="pt").input_ids.to(a.device)
    t0 = time.perf_counter()
    if a.engine:
        from ksa_b200.inference import KsaInferenceEngine
        eng = KsaInferenceEngine(model, max_len=ids.shape[1] + a.max_new_tokens + model.config.summary_chunk_size, batch=1)
        with torch.no_grad():
            out = eng.generate(ids, a.max_new_tokens, eos_id=model.config.eos_token_id,
                               temperature=0.0 if a.greedy else a.temperature, top_p=a.top_p)
    else:
        out = model.generate(ids, max_new_tokens=a.max_new_tokens, do_sample=not a.greedy, temperature=a.temperature,
                             top_p=a.top_p)
    if a.device.startswith("cuda"):
        torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    new = out[0, ids.shape[1]:]
    print(tok.decode(new, skip_special_tokens=True) if tok is not None else new.tolist())
    print(f"{new.numel()} new tokens in {dt:.2f} s ({new.numel() / dt:.1f} tok/s incl. prefill)")


if __name__ == "__main__":
    main()
