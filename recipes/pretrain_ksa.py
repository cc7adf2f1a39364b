#!/usr/bin/env python
"""Pre-training entry point for Qwen3 / Qwen3-KSA (counterpart of ``recipes/pretrain_kai_summary_unified.py``).

One process per GPU, launched with ``torchrun`` (``RANK / LOCAL_RANK / WORLD_SIZE``) or ``mpirun``
(``OMPI_COMM_WORLD_*``).  The flag set is a superset of the reference recipe's (``:79-261``); flags that configure
machinery this framework does not have (FlashAttention-2 selection, CPU offload, forward prefetch, resharding) are
accepted and ignored with a note, so the reference's launch scripts run unchanged.

Flow (``:326-1170`` of the reference): parse -> process group -> model config -> model on the meta device -> engine
(single GPU, or FSDP with the fused P2P kernels) -> optional weight / optimizer / dataloader resume -> loop of
``next batch -> labels -> step -> metrics -> periodic checkpoint``.  Differences that matter for speed: summary-token
layout is closed form (no per-step batch expansion), the loss head is the fused chunked linear+CE, the optimizer is
fused into the gradient reduction, and nothing in the step reads the device back except at the logging cadence.
"""
from __future__ import annotations

import argparse
import gc
import json
import os
import sys
import time

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def get_argument_parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser(description="Qwen3-KSA pre-training")
    a = p.add_argument
    # model / data
    a("--model-config", required=True, help="model JSON (reference format) or a preset name")
    a("--dataset-class", default="KaiMMapDataset")
    a("--dataset-config", default=None, help="dataset JSON; omit (or 'synthetic') for uniform-random token ids")
    a("--max-length", type=int, default=None, help="overrides the dataset's seq_length")
    a("--batch-size", type=int, default=1)
    a("--shuffle-buffer-size", type=int, default=0)
    a("--use-dataset-load-balance", action="store_true")
    a("--packing", action="store_true",
      help="batches carry cu_seqlens of packed documents: full-attention layers attend within documents only")
    # checkpoints
    a("--model-dir", default=None, help="HF directory to initialise the weights from")
    a("--checkpoint-dir", default=None)
    a("--checkpoint-id", default=None)
    a("--resume-weights", action="store_true")
    a("--resume-optimizer", action="store_true")
    a("--resume-dataloader", action="store_true")
    a("--save-checkpoint-per-step", type=int, default=0)
    a("--save-checkpoint-every-epoch", action="store_true")
    a("--async-checkpoint", action="store_true")
    a("--output-dir", required=True)
    a("--enable-dataset-checkpointing", action="store_true")
    # precision / sharding
    a("--model-dtype", default="bfloat16", choices=["bfloat16", "float16", "float32"])
    a("--cpu-offload", action="store_true")
    a("--fp32-weight", action="store_true", help="fp32 master weights (always on in this engine)")
    a("--fp32-reduce", action="store_true", help="fp32 gradient reduction (always on in this engine)")
    a("--reshard-after-forward", action="store_true")
    a("--prefetch-params-in-forward", action="store_true")
    a("--comm", default=None, choices=["fused", "collective"], help="FSDP back end (default: fused on GPUs)")
    a("--overlap", default="auto", choices=["auto", "stream", "gemm2"],
      help="fused back end: parameter gathers on a side stream, or inside the gate/up GEMM launches (auto: gemm2 for "
           "plain FSDP on 4 or more GPUs, else stream)")
    a("--no-cuda-graph", action="store_true")
    # optimisation
    a("--lr-scheduler-type", default="wsd", choices=["cosine", "cosine_v2", "wsd", "constant"])
    a("--num-warmup-steps", type=int, default=0)
    a("--num-decay-steps", type=int, default=0)
    a("--num-training-steps", type=int, default=1000)
    a("--num-epochs", type=int, default=1)
    a("--min-lr", type=float, default=0.0)
    a("--learning-rate", type=float, default=4e-4)
    a("--weight-decay", type=float, default=0.01)
    a("--beta1", type=float, default=0.9)
    a("--beta2", type=float, default=0.95)
    a("--clip-range", type=float, default=1.0)
    a("--use-flash-attention-2", action="store_true")
    a("--enable-gradient-checkpointing", action="store_true")
    a("--gradient-checkpointing-mode", default="full", choices=["full", "mlp"],
      help="with --enable-gradient-checkpointing: recompute whole layers, or only their feed-forward blocks")
    a("--gradient-accumulation-steps", type=int, default=1)
    a("--allow-random-init-params", default="", help="comma-separated parameter names that may be missing from "
      "--model-dir (or have another shape there) and keep their random initialisation")
    a("--skip-load-params", default="", help="comma-separated substrings: matching parameters are never loaded")
    a("--context-parallel-size", type=int, default=1)
    a("--chunked-loss-minibatch-size", type=int, default=2048)
    a("--disable-chunked-loss", action="store_true")
    # logging
    a("--logging-per-step", type=int, default=10)
    a("--monitor-datasource-loss", action="store_true")
    a("--no-tensorboard", action="store_true", help="do not write TensorBoard event files under <output-dir>/log")
    a("--num-workers", type=int, default=None,
      help="data-loading worker processes (default: the dataset JSON's num_workers for corpus data, 0 for synthetic)")
    a("--log-attn-stats", action="store_true")
    a("--comment", default="")
    a("--commit-id", default="")
    a("--seed", type=int, default=None)
    a("--enable-profile", action="store_true")
    a("--nvtx", action="store_true", help="NVTX ranges around data loading, the step and checkpoint saves")
    a("--step-timeout", type=float, default=1800.0,
      help="seconds without a finished step before the watchdog dumps all stacks (0 disables it)")
    a("--heartbeat-timeout", type=float, default=300.0,
      help="seconds without a peer's heartbeat before this rank stops between steps (multi-rank runs; 0 disables)")
    a("--resume-fallback", action="store_true",
      help="if the newest checkpoint is unfinished or unreadable, resume from the newest older complete one")
    a("--overfit-batches", type=int, default=0)
    # distillation
    a("--enable-distill", action="store_true")
    a("--distill-lm-loss-factor", type=float, default=1.0)
    a("--distill-kl-loss-factor", type=float, default=5.0)
    a("--distill-attn-mse-factor", type=float, default=5.0)
    a("--distill-attn-cos-factor", type=float, default=0.0)
    return p


def _env_rank():
    e = os.environ
    rank = int(e.get("RANK", e.get("OMPI_COMM_WORLD_RANK", "0")))
    world = int(e.get("WORLD_SIZE", e.get("OMPI_COMM_WORLD_SIZE", "1")))
    local = int(e.get("LOCAL_RANK", e.get("OMPI_COMM_WORLD_LOCAL_RANK", "0")))
    return rank, world, local


def _load_model_config(spec: str):
    from ksa_b200.config import get_preset, load_config, PRESETS
    return get_preset(spec) if spec in PRESETS else load_config(spec)


def _build_dataset(args, cfg, dp_rank: int, dp_size: int):
    from ksa_b200.data.mmap_dataset import KaiMMapDataset, SyntheticTokenDataset
    if not args.dataset_config or args.dataset_config == "synthetic":
        return SyntheticTokenDataset(cfg.vocab_size, args.max_length or 8192, args.seed or 0, dp_rank, args.batch_size)
    dc = json.load(open(args.dataset_config))
    if dc.pop("name", args.dataset_class) != "KaiMMapDataset":
        raise ValueError("only KaiMMapDataset (mmap token corpora) and synthetic data are supported")
    if args.max_length:
        dc["seq_length"] = args.max_length
    return KaiMMapDataset(rank=dp_rank, world_size=dp_size, **dc)


def train(args) -> dict:
    import torch
    import torch.distributed as dist
    from ksa_b200.data.mmap_dataset import make_labels
    from ksa_b200.losses import attention_cosine_loss, attention_mse_loss
    from ksa_b200.models import get_model_class
    from ksa_b200.models.base import load_full_state_dict
    from ksa_b200.parallel import groups
    from ksa_b200.training import checkpoint as ckpt
    from ksa_b200.training.activations import set_activation_checkpointing
    from ksa_b200.training.common import StepScheduler, freeze_params_by_pattern, to_dtype
    from ksa_b200.training.lr_schedulers import get_lr_lambda
    from ksa_b200.utils import print_rank_0, set_random_seed
    from ksa_b200.utils.metrics import CSVBackend, StdoutBackend, initialize_metrics
    from ksa_b200.utils.mfu import mfu as mfu_report

    gc.disable()
    rank, world, local = _env_rank()
    use_cuda = torch.cuda.is_available()
    if use_cuda:
        torch.cuda.set_device(local)
    device = torch.device("cuda", local) if use_cuda else torch.device("cpu")
    if world > 1 and not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29500")
        dist.init_process_group("nccl" if use_cuda else "gloo", rank=rank, world_size=world,
                                **({"device_id": device} if use_cuda else {}))
    cp = args.context_parallel_size
    if world > 1:
        groups.check_context_parallel_placement(cp, world)
        groups.initialize_model_parallel(cp)
        if groups.spans_nodes(world) and use_cuda:
            # peer memory ends at the node: across nodes the weights are gathered and the gradients reduced by NCCL
            if args.comm == "fused":
                raise SystemExit("--comm fused moves data through CUDA IPC peer memory and needs all ranks on one node; "
                                 f"this job has {groups.local_world_size(world)} of its {world} ranks per node")
            if args.comm is None:
                print_rank_0(f"[recipe] {world} ranks on nodes of {groups.local_world_size(world)}: FSDP over NCCL "
                             "collectives (--comm collective)")
                args.comm = "collective"
    dp_rank, dp_size = (groups.get_data_parallel_rank(), groups.get_data_parallel_world_size()) if world > 1 else (0, 1)
    if args.seed is not None:
        set_random_seed(args.seed)
    os.makedirs(args.output_dir, exist_ok=True)
    if rank == 0:
        json.dump(vars(args), open(os.path.join(args.output_dir, f"args-{int(time.time())}.json"), "w"), indent=2)
    # flags of the reference's CLI that mean nothing here: the attention kernels are this package's own, and the
    # next unit's parameters are always gathered one unit ahead
    if args.cpu_offload:
        print_rank_0("[recipe] --cpu-offload: fp32 master weights and Adam moments live in pinned host memory and pass "
                     "through a staging ring on the GPU for the update; the step runs eagerly")
    for flag in ("prefetch_params_in_forward", "use_flash_attention_2"):
        if getattr(args, flag):
            print_rank_0(f"[recipe] --{flag.replace('_', '-')} has no effect in this framework (accepted for compatibility)")

    cfg = _load_model_config(args.model_config)
    dtype = to_dtype(args.model_dtype) if use_cuda else torch.float32
    with torch.device("meta"):
        model = get_model_class(cfg.model_class)(cfg)
    model = model.to_empty(device=device).to(dtype)
    if args.model_dir:
        state = model.convert_hf_state_dict(ckpt.load_hf_checkpoint(args.model_dir))
        model.init_weights(seed=args.seed or 0)
        load_full_state_dict(model, state, args.allow_random_init_params, args.skip_load_params, verbose=print_rank_0)
    else:
        # every rank initialises from the same seed: identical weights with no broadcast (the reference initialises on
        # rank 0 and broadcasts parameter by parameter, muse/training/distributed.py:448-532)
        model.init_weights(seed=args.seed or 0)
    # --disable-chunked-loss: the head and the loss over the whole sequence at once (one chunk of logits)
    model.loss_chunk_tokens = (1 << 30) if args.disable_chunked_loss else args.chunked_loss_minibatch_size
    if args.enable_gradient_checkpointing:
        n = set_activation_checkpointing(model, model.get_checkpointable_module_classes(),
                                         mode=args.gradient_checkpointing_mode)
        print_rank_0(f"[recipe] activation checkpointing ({args.gradient_checkpointing_mode}) on {n} layers")
    if args.enable_distill:
        stats = freeze_params_by_pattern(model, ["summary_embedding", "_summary"])
        print_rank_0(f"[recipe] distillation: {stats['trainable']:,} trainable / {stats['frozen']:,} frozen parameters")

    lr_lambda = get_lr_lambda(args.lr_scheduler_type, num_warmup_steps=args.num_warmup_steps,
                              num_training_steps=args.num_training_steps, num_decay_steps=args.num_decay_steps,
                              base_lr=args.learning_rate, min_lr=args.min_lr)
    common = dict(lr=args.learning_rate, betas=(args.beta1, args.beta2), eps=1e-8, weight_decay=args.weight_decay,
                  clip_value=args.clip_range, lr_lambda=lr_lambda, grad_accum_steps=args.gradient_accumulation_steps,
                  cpu_offload=args.cpu_offload)
    if world > 1:
        from ksa_b200.parallel.fsdp import FsdpEngine, default_overlap
        if args.overlap == "auto":
            args.overlap = default_overlap(world, args.context_parallel_size, args.reshard_after_forward)
        engine = FsdpEngine(model, world_size=world, rank=rank, comm=args.comm, overlap=args.overlap,
                            reshard_after_forward=args.reshard_after_forward, **common)
    else:
        from ksa_b200.training.engine import TrainEngine
        engine = TrainEngine(model, **common)
    sched = StepScheduler(args.gradient_accumulation_steps, args.logging_per_step, args.save_checkpoint_per_step)

    dataset = _build_dataset(args, cfg, dp_rank, dp_size)
    seq_len = getattr(dataset, "seq_length", args.max_length or 8192)
    cp_rank = 0
    if cp > 1:
        # the sequence is cut into ``cp`` contiguous chunk-aligned shards; every rank of a group reads the same
        # sample (the dataset is indexed by data-parallel rank) and keeps its own slice
        from ksa_b200.parallel.cp import CpContext
        cp_rank = groups.get_context_parallel_rank()
        summary = bool(getattr(cfg, "summary_enabled", False))
        model.cp = CpContext(groups.get_context_parallel_group(), seq_len,
                             cfg.summary_chunk_size if summary else 128, cfg.summary_token_num if summary else 0,
                             cfg.num_kv_heads, cfg.head_dim, batch=args.batch_size,
                             device=device if use_cuda else None, dtype=dtype,
                             full_layers=not summary or any(not f for f in model._layer_is_summary()),
                             max_window=getattr(cfg, "summary_sliding_chunk_num", 8) if summary else 8,
                             n_heads=cfg.num_heads)
        if args.enable_distill:
            raise ValueError("distillation and context parallelism are not combined")
    checkpointer = ckpt.DistributedCheckpointer(async_save=args.async_checkpoint)
    step_offset = 0
    if args.checkpoint_dir and (args.resume_weights or args.resume_optimizer):
        app = ckpt.AppState(engine, sched, skip_optimizer=not args.resume_optimizer,
                            skip_training_state=not args.resume_optimizer)
        loaded = ckpt.load_checkpoint(app, checkpointer, args.checkpoint_dir, args.checkpoint_id,
                                      fallback=args.resume_fallback)
        if loaded is not None:
            print_rank_0(f"[recipe] resumed from step {loaded} of {args.checkpoint_dir}")
            step_offset = loaded - sched.global_step
            if args.resume_dataloader:
                ok = ckpt.load_dataloader_state(dataset, os.path.join(args.checkpoint_dir, ckpt.step_dir_name(loaded)))
                print_rank_0(f"[recipe] dataloader state {'restored' if ok else 'not found: starting the stream over'}")
    backends = [StdoutBackend(), CSVBackend(os.path.join(args.output_dir, "metrics.csv"))]
    if rank == 0 and not args.no_tensorboard:
        try:   # event files under <output-dir>/log, as the reference writes them (recipes/...:454-458)
            from ksa_b200.utils.metrics import TensorBoardBackend
            backends.append(TensorBoardBackend(os.path.join(args.output_dir, "log")))
        except Exception as e:  # noqa: BLE001 - tensorboard is optional
            print_rank_0(f"[recipe] TensorBoard logging is off: {type(e).__name__}: {e}")
    metrics = initialize_metrics(seq_len, world, args.logging_per_step, backends)
    source_monitor = None
    if args.monitor_datasource_loss:
        from ksa_b200.utils.metrics import SourceLossMonitor
        source_monitor = SourceLossMonitor()
    profiler = None
    if args.enable_profile:
        from torch.profiler import ProfilerActivity, profile, schedule
        profiler = profile(activities=[ProfilerActivity.CPU, ProfilerActivity.CUDA],
                           schedule=schedule(wait=50, warmup=1, active=10, repeat=1),
                           on_trace_ready=lambda p: p.export_chrome_trace(
                               os.path.join(args.output_dir, "torch_profile", f"{p.step_num}_w{rank}.json")))
        os.makedirs(os.path.join(args.output_dir, "torch_profile"), exist_ok=True)
        profiler.start()

    from ksa_b200.utils.tracing import StepTimer, nvtx_range
    from ksa_b200.utils.watchdog import FaultInjector, HeartbeatMonitor, StepWatchdog, check_device
    step_timer = StepTimer(device)
    watchdog = StepWatchdog(args.step_timeout).start() if args.step_timeout > 0 else None
    heartbeat = None
    if world > 1 and args.heartbeat_timeout > 0:
        from torch.distributed.distributed_c10d import _get_default_store
        heartbeat = HeartbeatMonitor(_get_default_store(), rank, world, args.heartbeat_timeout)
    faults = FaultInjector(rank=rank)

    # one CUDA graph per step on a single GPU; multi-GPU steps stay eager (see FsdpEngine.graphed_step)
    use_graph = use_cuda and world == 1 and not args.no_cuda_graph and not args.enable_distill \
        and not args.enable_gradient_checkpointing and not args.packing and not args.cpu_offload
    n_workers = args.num_workers if args.num_workers is not None else getattr(dataset, "loader_workers", 0)
    loader = dataset
    if n_workers > 0:
        from ksa_b200.data import ResumableLoader
        loader = ResumableLoader(dataset, num_workers=n_workers)
    data_iter = iter(loader)
    cached = []
    last_loss = None
    t_prev = t_log = time.perf_counter()
    while sched.global_step + step_offset < args.num_training_steps:
        # between steps, nothing in flight: stop here if a peer died rather than wait for it inside a collective
        try:
            faults.at_step(sched.micro_step)
        except Exception as e:
            if heartbeat is not None:
                heartbeat.report_failure(f"{type(e).__name__}: {e}")
            raise
        if heartbeat is not None:
            heartbeat.agree(sched.micro_step)
        with nvtx_range("data", args.nvtx):
            if args.overfit_batches and len(cached) >= args.overfit_batches:
                batch = cached[sched.micro_step % args.overfit_batches]
            else:
                batch = next(data_iter)
                if args.overfit_batches:
                    cached.append(batch)
        ids = batch["input_ids"]
        labels, _ = make_labels(ids, batch["loss_mask"])
        if "next_token" in batch:   # the corpus stores L+1 tokens: the last position has a real target
            labels[:, -1] = batch["next_token"]
        if cp > 1:                  # labels are shifted before the split, so a shard's last label is its successor's first token
            Ll = ids.shape[1] // cp
            ids = ids[:, cp_rank * Ll:(cp_rank + 1) * Ll].contiguous()
            labels = labels[:, cp_rank * Ll:(cp_rank + 1) * Ll].contiguous()
        if hasattr(model, "set_mix_coeff"):
            model.set_mix_coeff(sched.global_step + step_offset)
        with nvtx_range("step", args.nvtx):
            if args.enable_distill:
                loss = _distill_step(engine, model, ids.to(device), labels.to(device), args, attention_mse_loss,
                                     attention_cosine_loss)
            elif use_graph:
                loss = engine.graphed_step(ids.pin_memory() if use_cuda else ids,
                                           labels.pin_memory() if use_cuda else labels)
            else:
                kw = {}
                if args.packing and "cu_seqlens" in batch and batch["cu_seqlens"].numel() > 2 and cp == 1:
                    kw["cu_seqlens"] = batch["cu_seqlens"].to(device)     # documents stay apart in full-attention layers
                loss = engine.train_step(ids, labels, **kw)
        step_timer.tick()
        sched.step()
        if watchdog is not None:
            watchdog.beat()
        if heartbeat is not None:
            heartbeat.beat(sched.micro_step)
        if use_cuda and sched.should_logging():
            check_device()          # a bounded device-side wait that gave up shows here, as an exception
        metrics.loss.append(loss)
        if source_monitor is not None:
            source_monitor.add(batch, loss, int((labels != -100).sum()))
        metrics.tokens.append(ids.numel())
        metrics.samples.append(ids.shape[0])
        if sched.is_gradient_accumulation_boundary():
            metrics.grad_norm.append(engine.grad_norm())
            metrics.learning_rate.append(engine.current_lr(max(engine.step_count - 1, 0)))
            if use_cuda:
                torch.cuda.current_stream().synchronize() if sched.should_logging() else None
            now = time.perf_counter()
            metrics.step_time.append(now - t_prev)
            t_prev = now
        metrics.step()
        if sched.should_logging():
            scalars = metrics.write(sched.global_step + step_offset)
            last_loss = scalars.get("loss", last_loss)
            extra = {"perf/step_elapsed": time.perf_counter() - t_log}
            t_log = time.perf_counter()
            if getattr(cfg, "summary_mix_qkv", False) and hasattr(model, "layers"):
                extra["summary/mix_coeff"] = float(model.layers[0].attn.mix_coeff)
            if source_monitor is not None:
                extra.update(source_monitor.window())
            if rank == 0:
                for b in backends:
                    b.write(sched.global_step + step_offset, extra)
            if rank == 0 and "tokens_per_sec_per_gpu" in scalars:
                rep = mfu_report(scalars["tokens_per_sec_per_gpu"], cfg, seq_len,
                                 grad_checkpointing=args.enable_gradient_checkpointing, distill=args.enable_distill)
                print(f"[Metrics] step={sched.global_step + step_offset} | " +
                      " | ".join(f"{k}={v:.4g}" for k, v in rep.items()), flush=True)
        if args.save_checkpoint_per_step and sched.should_save_checkpoint() and not args.overfit_batches:
            gc.collect()
            step = sched.global_step + step_offset
            ckpt.save_checkpoint(ckpt.AppState(engine, sched), checkpointer, args.output_dir, step)
            if args.enable_dataset_checkpointing:
                ckpt.save_dataloader_state(loader, args.output_dir, step)
        if profiler is not None:
            profiler.step()
    checkpointer.wait()
    if profiler is not None:
        profiler.stop()
    if watchdog is not None:
        watchdog.stop()
    metrics.close()
    if getattr(model, "cp", None) is not None:
        model.cp.close()
    if hasattr(engine, "close"):
        engine.close()
    if world > 1:
        dist.barrier()
    timing = step_timer.summary(skip=min(3, max(sched.micro_step - 1, 0)))
    if rank == 0 and timing:
        print("[recipe] device time per micro-step: " + ", ".join(f"{k}={v:.3f}" for k, v in timing.items()), flush=True)
    return {"steps": sched.global_step + step_offset, "loss": last_loss, "step_ms": timing.get("median_ms")}


def _distill_step(engine, model, ids, labels, args, mse_fn, cos_fn):
    """Student forward (with summaries) + no-grad teacher forward (same weights, no summaries): LM + KL + attention
    matching losses (``recipes/pretrain_kai_summary_unified.py:967-1013``).  The losses run as the engine's
    ``step_fn``, inside its forward_backward, so gradient reduction, the optimizer and (under FSDP) the gathers of the
    refreshed weights are the engine's own."""
    import torch
    from ksa_b200.losses import ChunkedDistillLossComputer
    from ksa_b200.losses.distill import rms_normalize

    def step_fn(tokens, targets):
        model.skip_output_layer = True
        try:
            with torch.no_grad():
                t_hidden = model(tokens, collect_attn=True, use_summary=False)
                t_attn = list(model.last_attn_outputs)
            s_hidden = model(tokens, collect_attn=True)
            s_attn = list(model.last_attn_outputs)
        finally:
            model.skip_output_layer = False
        if getattr(model.config, "summary_distill_attention_norm", False):
            s_attn, t_attn = [rms_normalize(a) for a in s_attn], [rms_normalize(a) for a in t_attn]
        extra = args.distill_attn_mse_factor * mse_fn(s_attn, t_attn)
        if args.distill_attn_cos_factor:
            extra = extra + args.distill_attn_cos_factor * cos_fn(s_attn, t_attn)
        comp = ChunkedDistillLossComputer(model.lm_head_weight, args.chunked_loss_minibatch_size,
                                          args.distill_lm_loss_factor, args.distill_kl_loss_factor, enable_kl=True)
        out = comp.forward_and_backward(s_hidden, t_hidden, targets, engine.grad_accum_steps, extra_loss=extra)
        return out["total_loss"]

    return engine.train_step(ids, labels, step_fn=step_fn)


def main(argv=None):
    args = get_argument_parser().parse_args(argv)
    out = train(args)
    if _env_rank()[0] == 0:
        print(json.dumps({"done": True, **{k: (float(v) if v is not None else None) for k, v in out.items()}}))


if __name__ == "__main__":
    main()
