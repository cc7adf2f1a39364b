"""Reference arm of ``bench.py``: the unmodified reference (Muse trainer + its summary_attn / flash_attn_cute
wheels, installed under ``baseline/_ref``) on the same metric and configuration as our arm.

None of this repository's models, kernels or engine is on this path.  The harness drives the reference through
its public API in the order of its own training loop (``recipes/pretrain_kai_summary_unified.py:460-600`` for the
set-up, ``:855-1053`` for the step): ``load_config`` -> ``get_model_class`` on the meta device -> ``model.float()``
-> ``shard_model`` (FSDP2, bf16 parameters, fp32 reduction) -> ``initialize_model_params`` -> ``rope_init`` ->
``torch.optim.AdamW(model.get_optimizer_grouped_parameters(...))``; per step: labels from the original ids,
``maybe_build_summary_batch``, forward, ``CrossEntropyLoss``, backward, ``clip_grad_by_value``, optimizer step.

Environment shims (no reference source is edited): ``baseline/_ref`` is put on ``sys.path``; the wheel's
``flash_attn/cute`` directory is appended to the installed ``flash_attn`` package's ``__path__``; the process
group is created from torchrun's environment instead of OpenMPI's.  ``summary_attention_mode`` is ``kernel``
when a small call of ``summary_attn_func`` succeeds on this GPU, otherwise ``block`` (the reference's own PyTorch
mode); the JSON line names the back end that really served the call (``summary_attention_backend``: the wheel's CuTe
sm_100 kernel, its FlexAttention fallback, or ``block``), not the requested mode.

``--cp N --seq-len L`` runs the reference's own context parallelism (Ulysses all-to-all,
``muse/training/parallel.py:211-335``): ``initialize_model_parallel(N)``, the batch broadcast from the first rank
of each group, the per-rank slices of ids / position ids / labels / ``summary_mask`` with ``full_summary_mask`` kept
whole (``recipes/pretrain_kai_summary_unified.py:881-926``), and, as the reference's stage scripts do, activation
checkpointing from 32k tokens and the chunked lm_head + CE (``ChunkedDistillLossComputer``, 1024-token chunks) from
64k tokens (``examples/pretrain/run_pretrain_{32,64,128}k.sh``).
"""
from __future__ import annotations

import json
import os
import sys
import tempfile
import traceback

HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.path.join(HERE, "_ref")


def _model_json(mode: str, seq_len: int) -> dict:
    return {
        "__class__": "Qwen3SummaryAttentionConfig", "model_class": "Qwen3SummaryModel",
        "vocab_size": 151936, "embed_dim": 2048, "num_layers": 28, "num_heads": 16, "num_kv_heads": 8,
        "head_dim": 128, "intermediate_dim": 6144, "max_seq_len": max(131072, seq_len), "rope_base": 1000000,
        "norm_eps": 1e-6, "attn_dropout": 0.0, "attention_function": "flash_attention_2",
        "q_proj_bias": False, "k_proj_bias": False, "v_proj_bias": False, "q_norm": True, "k_norm": True,
        "tie_word_embeddings": False, "use_summary_attention": True, "summary_chunk_size": 128,
        "summary_token_num": 1, "summary_token_begin": 151936, "summary_sliding_chunk_num": 8,
        "summary_layer_freq": "([1]*3+[0]*1)*7", "summary_chunk_position_ids_type": "origin",
        "summary_token_position_ids_type": "last_chunk_slice_right", "summary_independent_parameters": True,
        "summary_attention_mode": mode,
    }


def _probe_kernel_mode(torch) -> str:
    """``kernel`` if the reference's CuTe-DSL summary attention runs forward+backward on this GPU, else the reason."""
    try:
        from summary_attn import summary_attn_func
        C, S, W, L = 128, 1, 8, 2048
        n = L + (L // C) * S
        q = torch.randn(1, n, 16, 128, device="cuda", dtype=torch.bfloat16, requires_grad=True)
        k = torch.randn(1, n, 16, 128, device="cuda", dtype=torch.bfloat16, requires_grad=True)
        v = torch.randn(1, n, 16, 128, device="cuda", dtype=torch.bfloat16, requires_grad=True)
        idx = torch.arange(n, device="cuda")
        summary_pos = idx[(idx % (C + S)) >= C]
        out = summary_attn_func(q, k, v, C, S, W, summary_pos=summary_pos)
        out = out[0] if isinstance(out, tuple) else out
        out.float().sum().backward()
        torch.cuda.synchronize()
        return "kernel"
    except Exception as e:  # noqa: BLE001 - any failure of the probe selects the reference's PyTorch mode
        return f"{type(e).__name__}: {str(e)[:160]}"


def run_reference_arm(args) -> dict:
    if not os.path.isdir(os.path.join(REF, "muse")):
        return {"impl": "reference", "unavailable": "baseline/_ref is empty: the reference was not installed on this machine"}
    if int(getattr(args, "cp", 1) or 1) > 1:
        # The path below is written out (it follows the reference's training loop), but its one run on this pool
        # (2 GPUs, 32768 tokens, --cp 2) ended in "CUDA error: an illegal memory access was encountered" inside the
        # reference's own step (record: profiles/reference_arm_cp2_32k_fault.md).  Reading the inputs against the
        # reference's recipe showed no mistake in them, so the path is not run again on shared GPUs.
        return {"impl": "reference",
                "unavailable": "the reference's context-parallel step (Ulysses all-to-all + activation checkpointing + its "
                               "FlexAttention fallback) raised 'CUDA error: an illegal memory access' on 2 x B200 at 32768 "
                               "tokens; not run again on this shared pool (profiles/reference_arm_cp2_32k_fault.md)"}
    try:
        return _run(args)
    except Exception as e:  # noqa: BLE001
        tb = traceback.format_exc().strip().splitlines()
        return {"impl": "reference", "unavailable": f"{type(e).__name__}: {str(e)[:200]} @ {tb[-3].strip() if len(tb) > 2 else ''}"}


def _run(args) -> dict:
    sys.path.insert(0, REF)
    import torch
    import torch.distributed as dist
    import torch.nn.functional as F
    import flash_attn
    flash_attn.__path__.append(os.path.join(REF, "flash_attn"))

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run")
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29533")
    os.environ.setdefault("RANK", "0")
    os.environ.setdefault("WORLD_SIZE", "1")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    dist.init_process_group("nccl", device_id=dev)
    from torch.distributed.device_mesh import init_device_mesh
    mesh = init_device_mesh("cuda", (world,))

    from muse.config import load_config
    from muse.models import get_model_class
    from muse.layers.summary_utils import maybe_build_summary_batch
    from muse.training.distributed import shard_model, initialize_model_params
    from muse.training.common import clip_grad_by_value, set_default_dtype
    cp = max(1, int(getattr(args, "cp", 1)))
    if world % cp:
        raise SystemExit(f"--cp {cp} does not divide {world} ranks")
    cp_group, cp_rank = None, 0
    if cp > 1:
        from muse.training.parallel import (broadcast_batch_tensors, get_context_parallel_group,
                                            get_context_parallel_rank, initialize_model_parallel)
        initialize_model_parallel(cp)
        cp_group, cp_rank = get_context_parallel_group(), get_context_parallel_rank()
    else:
        try:
            from muse.training.parallel import initialize_model_parallel
            initialize_model_parallel(1)
        except Exception:  # noqa: BLE001 - only needed for context parallelism
            pass

    probe = _probe_kernel_mode(torch)
    mode = "kernel" if probe == "kernel" else "block"
    backend = "block (the reference's PyTorch mode)"
    if mode == "kernel":
        import summary_attn.interface as sa_if
        backend = ("cute sm100 (flash_attn_cute wheel)" if sa_if._check_cute_available()
                   else "flex_attention fallback (torch.compile -> Triton)")
    L = args.seq_len
    grad_ckpt = L >= 32768          # the reference's 32k / 64k / 128k stage scripts pass --enable-gradient-checkpointing
    chunked_ce = L >= 65536         # ... and its 64k / 128k scripts use the chunked lm_head + CE
    with tempfile.NamedTemporaryFile("w", suffix=".json", delete=False) as f:
        json.dump(_model_json(mode, L), f)
    cfg = load_config(f.name)
    os.unlink(f.name)
    torch.manual_seed(0)
    with set_default_dtype("bfloat16"), torch.device("meta"):
        model = get_model_class(cfg.model_class)(cfg)
    if grad_ckpt:
        from muse.training.activations import set_activation_checkpointing
        set_activation_checkpointing(model, auto_wrap_policy=model.get_checkpointable_module_classes())
    model = model.float()                                     # --fp32-weight: fp32 master weights
    shard_model(model=model, cpu_offload=False, reshard_after_forward=False, dp_mesh=mesh, fp32_weight=True,
                prefetch_params_in_forward=False, fp32_reduce=True)
    dist.barrier()
    initialize_model_params(model)
    with torch.device(dev):
        for m in model.modules():
            if hasattr(m, "rope_init"):
                m.rope_init()
    chunked = None
    if chunked_ce:
        from muse.losses.chunked_distill_loss_computer import ChunkedDistillLossComputer
        model.model.skip_output_layer = True
        chunked = ChunkedDistillLossComputer(lm_head=model.model.output, minibatch_size=1024, lm_factor=1.0,
                                             kl_factor=0.0, enable_kl=False)
    loss_fn = torch.nn.CrossEntropyLoss(ignore_index=-100)
    opt = torch.optim.AdamW(model.get_optimizer_grouped_parameters(learning_rate=4e-4, weight_decay=0.1), lr=4e-4,
                            betas=(0.9, 0.95), eps=1e-8)

    g_cpu = torch.Generator().manual_seed(1234 + rank // cp)   # one sequence per context-parallel group
    n_batches = max(args.steps, 4)
    host = [torch.randint(0, cfg.vocab_size, (1, L), generator=g_cpu).pin_memory() for _ in range(n_batches)]
    resident = [t.to(dev) for t in host]

    def step(ids_src, read_loss: bool):
        ids = ids_src.to(dev, non_blocking=True)
        batch = {"input_ids": ids, "loss_mask": torch.ones_like(ids),
                 "position_ids": torch.arange(L, device=dev).unsqueeze(0),
                 "cu_seqlens": torch.tensor([0, L], device=dev, dtype=torch.int32)}
        shifted_ids = F.pad(batch["input_ids"][:, 1:], (0, 1), value=0)
        shifted_mask = F.pad(batch["loss_mask"][:, 1:], (0, 1), value=0)
        batch["labels"] = shifted_ids * shifted_mask + (-100) * (1 - shifted_mask)
        batch["loss_mask"] = shifted_mask.contiguous()
        batch, ctx = maybe_build_summary_batch(batch, cfg)
        ctx.curr_iteration = 0
        if cp > 1:
            broadcast_batch_tensors(batch, cp_group)
            n = batch["input_ids"].shape[1] // cp
            batch["input_ids"] = batch["input_ids"][:, cp_rank * n:(cp_rank + 1) * n].contiguous()
            if batch.get("position_ids") is not None:
                batch["position_ids"] = batch["position_ids"][:, cp_rank * n:(cp_rank + 1) * n].contiguous()
            m = batch["labels"].shape[1] // cp
            batch["labels"] = batch["labels"][:, cp_rank * m:(cp_rank + 1) * m].contiguous()
            batch["loss_mask"] = batch["loss_mask"][:, cp_rank * m:(cp_rank + 1) * m].contiguous()
            ctx.full_summary_mask = ctx.summary_mask
            k = ctx.summary_mask.shape[1] // cp
            ctx.summary_mask = ctx.summary_mask[:, cp_rank * k:(cp_rank + 1) * k].contiguous()
            ctx.position_ids = ctx.position_ids[:, cp_rank * k:(cp_rank + 1) * k].contiguous()
        else:
            ctx.full_summary_mask = ctx.summary_mask
        labels = batch["labels"]
        out = model(tokens=batch["input_ids"], cu_seqlens=batch.get("cu_seqlens"), input_pos=batch.get("position_ids"),
                    summary_ctx=ctx)
        if isinstance(out, tuple):
            out = out[0]
        if chunked is not None:
            loss = chunked.forward_and_backward(out, None, labels, gradient_accumulation_steps=1)["total_loss"]
        else:
            loss = loss_fn(out.reshape(-1, out.size(-1)), labels.reshape(-1))
            loss.backward()
        clip_grad_by_value(model, 1.0)
        opt.step()
        opt.zero_grad()
        return loss.item() if read_loss else loss

    def barrier():
        dist.barrier()
        torch.cuda.synchronize(dev)

    from bench import ClockSampler, METRIC, MODEL_NAME  # clock sampling helper only
    for i in range(max(args.warmup, 3)):
        loss0 = step(resident[i % n_batches], True)
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(args.steps):
        step(resident[i % n_batches], False)
    e1.record()
    barrier()
    ms_dev = e0.elapsed_time(e1)
    barrier()
    e2, e3 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e2.record()
    last = 0.0
    for i in range(args.steps):
        last = step(host[i % n_batches], True)
    e3.record()
    barrier()
    ms_e2e = e2.elapsed_time(e3)
    clocks = sampler.stop() if rank == 0 else {}
    t = torch.tensor([ms_dev, ms_e2e], device=dev, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_dev, ms_e2e = t.tolist()
    dist.destroy_process_group()
    tokens = (world // cp) * L * args.steps
    out = {
        "metric": METRIC, "value": tokens / (ms_dev / 1e3), "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms_dev / args.steps, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic uniform-random token ids, random-init weights",
        "impl": "reference",
        "config": {"model": MODEL_NAME, "global_batch": world // cp, "seq_len": L,
                   "parallelism": f"fsdp{world}" + (f"+cp{cp} (Ulysses all-to-all)" if cp > 1 else ""),
                   "summary_attention_mode": mode, "summary_attention_backend": backend,
                   "kernel_mode_probe": probe, "full_attention": "flash_attention_2",
                   "activation_checkpointing": grad_ckpt, "chunked_ce": chunked_ce,
                   "l2": "working set exceeds L2; no explicit flush"},
        "clocks": clocks,
        "e2e": {"value": tokens / (ms_e2e / 1e3), "unit": "tokens/s", "ms_per_step": ms_e2e / args.steps,
                "h2d_bytes_per_step": L * 8, "d2h_bytes_per_step": 4},   # every rank of a group copies the whole sequence
        "gpu_launches": 0, "loss_first": loss0, "loss_last": last,
    }
    return out if rank == 0 else None
