#!/usr/bin/env python
"""Headline benchmark: Qwen3-1.9B-KSA pretraining throughput at 8k context (text tokens per second, whole job).

    python bench.py --gpus 1 --steps 8 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29511 \
        bench.py --gpus 8 --steps 8 --warmup 3
    python bench.py --impl reference ...      # the unmodified reference from baseline/_ref, same metric and config

Model: 28 layers (3 summary-attention : 1 full), hidden 2048, 16 Q / 8 KV heads x 128, SwiGLU 6144,
vocab 151936, untied embeddings; chunk 128 + 1 summary token, window 8 chunks; random init N(0, 0.02).
Work per step and per GPU: one sequence of 8192 uniform-random token ids (weak scaling), full
forward + backward + AdamW (fp32 master weights, beta 0.9/0.95, wd 0.1), bf16 compute.

Timing: W untimed warm-up steps, then exactly K steps between barrier + synchronize on both sides, CUDA
events on the launching stream, max over ranks.  The step's working set (tens of GB of weights, optimizer
state and activations) is far larger than the 126 MB L2, so no explicit flush is needed between steps.
``value`` is measured with the step's inputs already resident on the device; ``e2e`` repeats the K steps
through ``TrainEngine.graphed_step`` with, every step, a host->device copy of the token ids and labels from
pinned memory and a device->host read of the loss.  SM clocks and throttle reasons are sampled with
nvidia-smi during the timed region.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

MODEL_NAME = "Qwen3-1.9B-KSA"
SEQ_LEN = 8192
METRIC = "train_text_tokens_per_sec"


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=8)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--seq-len", type=int, default=SEQ_LEN)
    ap.add_argument("--preset", default="qwen3-1.9b-ksa")
    ap.add_argument("--cp", type=int, default=1,
                    help="context-parallel size: --seq-len is the whole sequence, split over groups of this many ranks")
    ap.add_argument("--cp-full-layers", default="auto", choices=["auto", "ulysses", "halo"],
                    help="full-attention layers under --cp: head-parallel resharding or staged earlier keys")
    ap.add_argument("--no-graph", action="store_true", help="launch kernels eagerly instead of replaying a CUDA graph")
    ap.add_argument("--comm", default=None, choices=["fused", "collective"],
                    help="multi-GPU back end: fused P2P kernels (default) or NCCL collectives (A/B baseline)")
    ap.add_argument("--overlap", default="auto", choices=["auto", "stream", "gemm2"],
                    help="fused back end: parameter gathers on a side stream, or inside the gate/up GEMM launches "
                         "(auto: gemm2 for plain FSDP on 4 or more GPUs, where it measured faster, else stream)")
    ap.add_argument("--reshard", action="store_true",
                    help="ZeRO-3: keep only 1/N of the bf16 weights resident and re-gather units for backward")
    ap.add_argument("--cpu-offload", action="store_true",
                    help="fp32 master weights and Adam moments in pinned host memory (staged through the GPU per unit)")
    return ap.parse_args()


class ClockSampler:
    """nvidia-smi clock / throttle sampling in the background (read-only queries)."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.proc = None
        self.path = None

    def start(self):
        try:
            f = tempfile.NamedTemporaryFile("w", suffix=".csv", delete=False)
            self.path = f.name
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.gpu_index), f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=f, stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        try:
            for line in open(self.path):
                parts = [p.strip() for p in line.split(",")]
                if len(parts) < 9:
                    continue
                try:
                    sm.append(float(parts[1])); mx.append(float(parts[2]))
                except ValueError:
                    continue
                for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"),
                                     parts[5:9]):
                    if val.lower().startswith("active"):
                        reasons.add(name)
            os.unlink(self.path)
        except Exception:
            pass
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def run_ours(args) -> dict:
    import torch
    import torch.distributed as dist
    from ksa_b200.config import get_preset
    from ksa_b200.models import get_model_class
    from ksa_b200.ops import _lib

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    cfg = get_preset(args.preset)
    torch.manual_seed(0)
    with torch.device("meta"):
        model = get_model_class(cfg.model_class)(cfg)
    model = model.to_empty(device=dev).to(torch.bfloat16)
    gen = torch.Generator(device=dev).manual_seed(0)
    with torch.no_grad():
        for p in model.parameters():
            if p.dim() >= 2:
                p.normal_(0.0, 0.02, generator=gen)
            else:
                p.fill_(1.0)

    if world > 1:
        from ksa_b200.parallel.fsdp import FsdpEngine as Engine, default_overlap
        if args.overlap == "auto":
            args.overlap = default_overlap(world, args.cp, args.reshard)
        extra = dict(world_size=world, rank=rank, comm=args.comm, overlap=args.overlap,
                     reshard_after_forward=args.reshard)
    else:
        from ksa_b200.training.engine import TrainEngine as Engine
        extra = {}
    engine = Engine(model, lr=4e-4, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1, clip_value=1.0,
                    cpu_offload=args.cpu_offload, **extra)

    B, L = 1, args.seq_len
    cp, dp = args.cp, world // max(args.cp, 1)
    if cp > 1:
        from ksa_b200.parallel.cp import CpContext
        if world % cp:
            raise SystemExit(f"--cp {cp} does not divide {world} ranks")
        groups = [dist.new_group(list(range(i * cp, (i + 1) * cp))) for i in range(dp)] if dp > 1 else [dist.group.WORLD]
        full_layers = any(not f for f in model._layer_is_summary())
        model.cp = CpContext(groups[rank // cp], L, cfg.summary_chunk_size, cfg.summary_token_num, cfg.num_kv_heads,
                             cfg.head_dim, batch=B, device=dev, full_layers=full_layers,
                             max_window=cfg.summary_sliding_chunk_num, n_heads=cfg.num_heads,
                             full_layer_mode=args.cp_full_layers)
    g_cpu = torch.Generator().manual_seed(1234 + rank // cp)     # one sequence per context-parallel group
    n_batches = max(args.steps, 4)
    host_tokens = [torch.randint(0, cfg.vocab_size, (B, L + 1), generator=g_cpu) for _ in range(n_batches)]
    if cp > 1:   # this rank's contiguous shard of inputs and (already shifted) labels
        Ll, r = L // cp, rank % cp
        host_tokens = [torch.cat([t[:, r * Ll:(r + 1) * Ll], t[:, (r + 1) * Ll:(r + 1) * Ll + 1]], dim=1) for t in host_tokens]
    host_in = [t[:, :-1].contiguous().pin_memory() for t in host_tokens]
    host_lab = [t[:, 1:].contiguous().pin_memory() for t in host_tokens]
    dev_in = [t.to(dev) for t in host_in]
    dev_lab = [t.to(dev) for t in host_lab]

    # one CUDA graph for the whole step on one GPU; the multi-GPU step stays eager (its communication kernels wait on
    # other GPUs' flags from a side stream, an ordering that a graph replay does not promise to keep)
    use_graph = not args.no_graph and world == 1 and not args.cpu_offload
    step_fn = engine.graphed_step if use_graph else engine.train_step

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    for i in range(max(args.warmup, 3)):
        loss = step_fn(dev_in[i % n_batches], dev_lab[i % n_batches])
    torch.cuda.synchronize(dev)
    _lib.check_status()
    loss0 = float(loss)

    # launches of this library's kernels per step (counted while one eager step runs)
    launches_per_step = _lib.count_launches(lambda: engine.train_step(dev_in[0], dev_lab[0]))
    torch.cuda.synchronize(dev)

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    # ---- device-timed: inputs resident on the device
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(args.steps):
        loss = step_fn(dev_in[i % n_batches], dev_lab[i % n_batches])
    e1.record()
    barrier()
    ms_dev = e0.elapsed_time(e1)
    # ---- end to end: pinned host inputs -> device each step, loss read back each step
    barrier()
    e2, e3 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e2.record()
    last = 0.0
    for i in range(args.steps):
        loss = step_fn(host_in[i % n_batches], host_lab[i % n_batches])
        last = loss.item()
    e3.record()
    barrier()
    ms_e2e = e2.elapsed_time(e3)
    clocks = sampler.stop() if rank == 0 else {}
    _lib.check_status()

    t = torch.tensor([ms_dev, ms_e2e], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_dev, ms_e2e = t.tolist()
    tokens_per_step = dp * B * L
    value = tokens_per_step * args.steps / (ms_dev / 1e3)
    e2e_value = tokens_per_step * args.steps / (ms_e2e / 1e3)
    h2d = 2 * B * (L // cp) * 8
    out = {
        "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms_dev / args.steps, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic uniform-random token ids, random-init weights",
        "impl": "ours",
        "config": {"model": MODEL_NAME, "global_batch": dp * B, "seq_len": L,
                   "parallelism": (f"fsdp{world}" + (f"+cp{cp}" if cp > 1 else "")) if world > 1 else "single",
                   "layers": cfg.num_layers,
                   "chunk": cfg.summary_chunk_size, "window_chunks": cfg.summary_sliding_chunk_num, "optimizer": "AdamW fp32 master",
                   "l2": "working set (weights+optimizer state+activations, >30 GB) exceeds L2; no explicit flush",
                   "cuda_graph": use_graph, "comm": getattr(engine, "comm", "none"),
                   "overlap": getattr(engine, "overlap", "none"),
                   "reshard_after_forward": bool(getattr(engine, "reshard", False)),
                   "cpu_offload": bool(args.cpu_offload),
                   "offload_bytes_each_way_per_step": sum(u.host_state.numel() * 4 for u in engine.units)
                   if args.cpu_offload else 0},
        "clocks": clocks,
        "e2e": {"value": e2e_value, "unit": "tokens/s", "ms_per_step": ms_e2e / args.steps,
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4},
        "gpu_launches": launches_per_step * args.steps,
        "loss_first": loss0, "loss_last": last,
    }
    if world > 1:
        if model.cp is not None:
            model.cp.close()
        if hasattr(engine, "close"):
            engine.close()
        dist.destroy_process_group()
    return out if rank == 0 else None


def run_reference(args) -> dict:
    from baseline.reference_arm import run_reference_arm
    return run_reference_arm(args)


def main():
    args = parse_args()
    if args.impl == "reference":
        out = run_reference(args)
    else:
        out = run_ours(args)
    if out is not None:
        print(json.dumps(out), flush=True)


if __name__ == "__main__":
    main()
