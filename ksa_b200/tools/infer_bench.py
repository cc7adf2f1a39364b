"""Prefill + greedy-decode benchmark of the inference engine (random-init weights, uniform-random prompt).

    python -m ksa_b200.tools.infer_bench --preset ksa-4b --prompt-len 131072 --decode 512 --batch 1
    python -m torch.distributed.run --nproc-per-node 4 --master-addr 127.0.0.1 -m ksa_b200.tools.infer_bench \\
        --preset ksa-4b --prompt-len 131072 --decode 512 --batch 16          # tensor parallel over 4 GPUs

Times are CUDA-event times on the launching stream, maximum over ranks; one warm-up prefill and a few warm-up decode
steps run first.  Prints one JSON line: prefill tokens/s (prompt tokens of all sequences / prefill time), decode
tokens/s (batch x steps / decode time) and milliseconds per decode step.
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist

from ..config import get_preset
from ..inference.engine import KsaInferenceEngine
from ..models import get_model_class
from ..ops import _lib


def _random_model(cfg, device, dtype, seed: int):
    with torch.device("meta"):
        model = get_model_class(cfg.model_class)(cfg)
    model = model.to_empty(device=device).to(dtype)
    gen = torch.Generator(device=device).manual_seed(seed)
    with torch.no_grad():
        for p in model.parameters():
            if p.dim() >= 2:
                p.normal_(0.0, 0.02, generator=gen)
            else:
                p.fill_(1.0)
    return model


def main(argv=None) -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--preset", default="ksa-4b")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"],
                    help="reference: the reference's own HF template through AutoModelForCausalLM + generate "
                         "(batch 1, one GPU); prints an `unavailable` line where it cannot run")
    ap.add_argument("--prompt-len", type=int, default=131072)
    ap.add_argument("--decode", type=int, default=512)
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--warmup-decode", type=int, default=8)
    ap.add_argument("--no-warmup-prefill", action="store_true")
    ap.add_argument("--tp-two-phase-min", type=int, default=None,
                    help="smallest group that uses the reduce-scatter + gather form for prefill (default 3)")
    ap.add_argument("--tp-separate-gather", action="store_true",
                    help="gather the normalised rows with kernels of their own instead of inside the projection "
                         "that consumes them (for A/B runs)")
    ap.add_argument("--tp-pull-partials", action="store_true",
                    help="the reduce-scatter pulls the partial blocks from the peers instead of the row-parallel GEMMs "
                         "scattering them into the owners' memory from the epilogue (for A/B runs)")
    a = ap.parse_args(argv)
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    if a.impl == "reference":
        import sys
        root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
        sys.path.insert(0, root)
        from baseline.reference_infer_arm import run_reference_infer_arm
        if rank == 0:
            print(json.dumps(run_reference_infer_arm(a.prompt_len, a.decode, a.batch, world)), flush=True)
        return
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    cfg = get_preset(a.preset)
    C, S = cfg.summary_chunk_size, cfg.summary_token_num
    B, L = a.batch, a.prompt_len
    tp = None
    local_cfg = cfg
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
        from ..parallel.tp import TpContext, tp_local_config
        rows = B * (L + (L // C) * S)
        tp = TpContext(dist.group.WORLD, cfg.embed_dim, max_rows=rows, device=dev,
                       two_phase_min_size=a.tp_two_phase_min, fused_gather=False if a.tp_separate_gather else None,
                       push_partials=False if a.tp_pull_partials else None)
        local_cfg = tp_local_config(cfg, world)
    model = _random_model(local_cfg, dev, torch.bfloat16, seed=0)   # same seed: replicated tensors agree across ranks
    if tp is not None:
        model.tp = tp
        if model.output is not None and cfg.vocab_size % world == 0:     # vocabulary-parallel head
            n = cfg.vocab_size // world
            model.output.weight = torch.nn.Parameter(model.output.weight[rank * n:(rank + 1) * n].clone())
    eng = KsaInferenceEngine(model, max_len=L + a.decode + a.warmup_decode + C, batch=B)
    g = torch.Generator().manual_seed(1)
    prompt = torch.randint(0, min(cfg.vocab_size, 150000), (B, L), generator=g).to(dev)

    def sync_max(ms: float) -> float:
        if world == 1:
            return ms
        t = torch.tensor([ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t)

    def timed(fn):
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        out = fn()
        e.record()
        torch.cuda.synchronize()
        return out, sync_max(s.elapsed_time(e))

    if not a.no_warmup_prefill:
        eng.prefill(prompt)
    logits, ms_prefill = timed(lambda: eng.prefill(prompt))
    nxt = logits.argmax(-1)
    for _ in range(a.warmup_decode if a.decode > 0 else 0):
        nxt = eng.decode_step(nxt).argmax(-1)

    def decode():
        t = nxt
        for _ in range(a.decode):
            t = eng.decode_step(t).argmax(-1)
        return t
    ms_decode = timed(decode)[1] if a.decode > 0 else None
    _lib.check_status()
    if rank == 0:
        steps = max(a.decode, 1)
        print(json.dumps({
            "model": a.preset, "tp": world, "batch": B, "prompt_len": L, "decode_steps": a.decode, "dtype": "bf16",
            "tp_prefill": (None if tp is None else
                           {"two_phase": bool(tp.two_phase_rows), "fused_gather": tp.fused_gather,
                            "push_partials": tp.push_partials}),
            "prefill_ms": ms_prefill, "prefill_tokens_per_s": B * L / (ms_prefill / 1e3),
            "decode_ms_per_step": None if ms_decode is None else ms_decode / steps,
            "decode_tokens_per_s": None if ms_decode is None else B * a.decode / (ms_decode / 1e3),
            "kv_cache_gb_per_gpu": eng.cache_bytes() / 1e9, "data": "uniform random prompt, random-init weights"}),
            flush=True)
    if tp is not None:
        tp.close()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
