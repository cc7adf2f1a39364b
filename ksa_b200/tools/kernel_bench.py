"""Micro-benchmarks of the sm_100a kernels against their rooflines (CUDA events, L2 flushed between iterations).

    python -m ksa_b200.tools.kernel_bench gemm --m 8192 --n 4096 --k 2048
    python -m ksa_b200.tools.kernel_bench attn --seq 8192 [--causal] [--bwd]
    python -m ksa_b200.tools.kernel_bench decode --cap 131072 --batch 16
    python -m ksa_b200.tools.kernel_bench norm --rows 8256 --dim 2048
    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 -m ksa_b200.tools.kernel_bench \
        cp-attn --seq 32768 --bwd          # context-parallel attention: one shard per rank, max over ranks
    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 -m ksa_b200.tools.kernel_bench comm
    python -m ksa_b200.tools.kernel_bench comm --world 2      # the same kernels over buffers of one GPU
    python -m torch.distributed.run --nproc-per-node 4 --master-addr 127.0.0.1 -m ksa_b200.tools.kernel_bench \
        ag-gemm --gemm-m 33024 --gemm-n 1536 --gemm-k 2560   # all-gather -> GEMM in one launch vs gather kernel + GEMM
    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 -m ksa_b200.tools.kernel_bench \
        gemm-rs --gemm-m 33024 --gemm-k 2048 --dim 2560      # GEMM -> reduce-scatter: scattered by the epilogue vs pulled
    python -m ksa_b200.tools.kernel_bench gemm --pair --scatter-world 4 --m 33024 --n 2560 --k 2048   # the same GEMM alone

Each line reports the median time, the achieved TFLOP/s or GB/s and, when ``MEASURED_PEAKS.json`` sits at the
repository root, the fraction of the measured peak (cuBLAS bf16 burst / STREAM-style copy).  ``--iters 1 --warmup 1
--no-flush`` gives a short, fixed launch sequence suitable for a profiler capture of one kernel.
"""
from __future__ import annotations

import argparse
import json
import os

import torch

from .. import ops
from ..ops import _lib
from ..ops.layout import count_attended_pairs

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def peaks() -> dict:
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return {"tflops": d.get("bf16_tflops"), "gbs": d.get("hbm_gbs"), "src": "measured"}
    return {"tflops": 1590.0, "gbs": 6650.0, "src": "fallback"}


def timeit(fn, iters: int, warmup: int, flush: bool) -> float:
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    buf = torch.empty(256 << 20, dtype=torch.uint8, device="cuda") if flush else None
    times = []
    for _ in range(iters):
        if buf is not None:
            buf.zero_()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        times.append(s.elapsed_time(e))
    times.sort()
    return times[len(times) // 2]


def report(name: str, ms: float, flops: float = 0.0, bytes_: float = 0.0) -> None:
    pk = peaks()
    parts = [f"{name}: {ms:.4f} ms"]
    if flops:
        tf = flops / ms / 1e9
        parts.append(f"{tf:.0f} TFLOP/s ({tf / pk['tflops']:.2f} of {pk['src']} {pk['tflops']:.0f})")
    if bytes_:
        gb = bytes_ / ms / 1e6
        parts.append(f"{gb:.0f} GB/s ({gb / pk['gbs']:.2f} of {pk['src']} {pk['gbs']:.0f})")
    print(" | ".join(parts), flush=True)


def bench_gemm(a) -> None:
    M, N, K = a.m, a.n, a.k
    A = torch.randn((K, M) if a.a_mn else (M, K), device="cuda").bfloat16()
    B = torch.randn((K, N) if a.b_mn else (N, K), device="cuda").bfloat16()
    C = torch.empty(M, N, device="cuda", dtype=torch.float32 if a.fp32_out else torch.bfloat16)
    if a.scatter_world > 0:
        # GEMM -> reduce-scatter, producer side, as one process: the row blocks go to --scatter-world buffers of this GPU
        import ctypes
        W = a.scatter_world
        shard = (M + W - 1) // W
        outs = [torch.empty(shard, N, device="cuda", dtype=torch.bfloat16) for _ in range(W)]
        ptrs = (ctypes.c_void_p * W)(*[o.data_ptr() for o in outs])
        ms = timeit(lambda: _lib.call("ksa_gemm2_scatter_bf16", A, B, M, N, K, A.stride(0), B.stride(0), N, ptrs, W, shard),
                    a.iters, a.warmup, not a.no_flush)
        report(f"gemm {M}x{N}x{K} scattering its row blocks to {W} local buffers (CTA pairs, TMA stores)", ms,
               flops=2.0 * M * N * K)
        return
    ms = timeit(lambda: ops.gemm(A, B, a_mn_major=a.a_mn, b_mn_major=a.b_mn, out=C, pair=a.pair), a.iters, a.warmup,
                not a.no_flush)
    report(f"gemm {M}x{N}x{K} a_mn={int(a.a_mn)} b_mn={int(a.b_mn)}" + (" (CTA pairs)" if a.pair else ""), ms,
           flops=2.0 * M * N * K)
    if a.compare:
        Am, Bm = (A.t() if a.a_mn else A), (B if a.b_mn else B.t())
        Cb = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        ms2 = timeit(lambda: torch.matmul(Am, Bm, out=Cb), a.iters, a.warmup, not a.no_flush)
        report("  cuBLAS (torch.matmul)", ms2, flops=2.0 * M * N * K)


def bench_gemv(a) -> None:
    """Decode-shaped projection: ``--m`` activation rows (<= 16) against an ``[n, k]`` weight; bytes = the weight."""
    M, N, K = a.m, a.n, a.k
    A = torch.randn(M, K, device="cuda").bfloat16()
    B = torch.randn(N, K, device="cuda").bfloat16()
    C = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
    ms = timeit(lambda: ops.gemm(A, B, out=C), a.iters, a.warmup, not a.no_flush)
    report(f"skinny gemm {M}x{N}x{K}", ms, bytes_=2.0 * N * K)


def bench_attn(a) -> None:
    B, Hq, Hkv, D, C, S, W, L = a.batch, a.hq, a.hkv, a.dim, a.chunk, a.nsum, a.window, a.seq
    Ns = 0 if a.causal else (L // C) * S
    R = B * (L + Ns)
    qkv = torch.randn(R, (Hq + 2 * Hkv) * D, device="cuda").bfloat16().requires_grad_(a.bwd)
    kw = {} if a.causal else dict(chunk=C, n_sum=S, window=W)
    pairs = L * (L + 1) // 2 if a.causal else count_attended_pairs(L, C, S, W)
    fwd_flops = 4.0 * D * Hq * pairs * B
    out = [None]

    def fwd():
        out[0] = ops.attention_packed(qkv, B, L, Ns, Hq, Hkv, D, **kw)
    ms_f = timeit(fwd, a.iters, a.warmup, not a.no_flush)
    kind = "causal" if a.causal else f"ksa C{C} S{S} W{W}"
    report(f"attention fwd {kind} L{L} {Hq}q/{Hkv}kv d{D}", ms_f, flops=fwd_flops)
    if a.bwd:
        g = torch.randn_like(out[0])

        def fb():
            fwd()
            out[0].backward(g)
        ms_fb = timeit(fb, a.iters, a.warmup, not a.no_flush)
        report(f"attention bwd {kind} L{L} (fwd+bwd minus fwd; useful FLOPs = 2.5x fwd)", ms_fb - ms_f,
               flops=2.5 * fwd_flops)
    if a.compare_ref:
        _compare_reference_attention(a, fwd_flops)


def _compare_reference_attention(a, fwd_flops: float) -> None:
    """Same shapes on other implementations, same GPU, same timing: flash_attn 2.x (dense causal only) and the
    reference's own sm_100 kernels from its wheels (``baseline/reference_kernels.py``; one GPU only)."""
    import sys
    sys.path.insert(0, ROOT)
    from baseline import reference_kernels as rk
    B, Hq, Hkv, D, C, S, W, L = a.batch, a.hq, a.hkv, a.dim, a.chunk, a.nsum, a.window, a.seq
    mk = lambda T, H: torch.randn(B, T, H, D, device="cuda").bfloat16().requires_grad_(a.bwd)

    def run(name, fn, make_inputs):
        try:
            xs = make_inputs()
            out = [None]

            def f():
                out[0] = fn(*xs)
            ms_f = timeit(f, a.iters, a.warmup, not a.no_flush)
            report(f"  {name} fwd", ms_f, flops=fwd_flops)
            if a.bwd:
                g = torch.randn_like(out[0])

                def fb():
                    f()
                    out[0].backward(g)
                ms_fb = timeit(fb, a.iters, a.warmup, not a.no_flush)
                report(f"  {name} bwd (fwd+bwd minus fwd)", ms_fb - ms_f, flops=2.5 * fwd_flops)
        except BaseException as e:  # noqa: BLE001 - a JIT compilation failure must not end the comparison
            print(f"  {name}: unavailable: {' '.join(f'{type(e).__name__}: {e}'.split())[:300]}", flush=True)

    if a.causal:
        try:
            from flash_attn import flash_attn_func as fa2
            run("flash_attn 2.x causal", lambda q, k, v: fa2(q, k, v, causal=True), lambda: (mk(L, Hq), mk(L, Hkv), mk(L, Hkv)))
        except BaseException as e:  # noqa: BLE001
            print(f"  flash_attn 2.x: unavailable: {type(e).__name__}: {e}", flush=True)
        fn, why = rk.dense_causal()
        if fn is None:
            print(f"  reference sm_100 causal (flash_attn_cute wheel): unavailable: {why}", flush=True)
        else:
            run("reference sm_100 causal (flash_attn_cute wheel)", fn, lambda: (mk(L, Hq), mk(L, Hkv), mk(L, Hkv)))
        return
    fn, why = rk.summary_attention(C, S, W)
    if fn is None:
        print(f"  reference sm_100 summary attention: unavailable: {why}", flush=True)
        return
    T = L + (L // C) * S                     # the reference's interleaved layout, K/V expanded to the query heads
    idx = torch.arange(T, device="cuda")
    summary_pos = idx[(idx % (C + S)) >= C]
    run("reference sm_100 summary attention (wheels, 256x128 lists)",
        lambda q, k, v: fn(q, k, v, summary_pos), lambda: (mk(T, Hq), mk(T, Hq), mk(T, Hq)))


def bench_decode(a) -> None:
    from ..inference.engine import _decode_attention
    B, Hq, Hkv, D, cap = a.batch, a.hq, a.hkv, a.dim, a.cap
    q = torch.randn(B, 1, Hq, D, device="cuda").bfloat16()
    k = torch.randn(B, Hkv, cap, D, device="cuda").bfloat16()
    v = torch.randn_like(k)
    start = torch.zeros(B, 1, dtype=torch.int32, device="cuda")
    length = torch.full((B, 1), cap, dtype=torch.int32, device="cuda")
    ms = timeit(lambda: _decode_attention(q, k, v, start, length, D ** -0.5), a.iters, a.warmup, not a.no_flush)
    report(f"decode attention B{B} {Hq}q/{Hkv}kv cap {cap}", ms, bytes_=2.0 * k.numel() * 2)


def bench_norm(a) -> None:
    rows, D = a.rows, a.dim
    x, d = torch.randn(rows, D, device="cuda").bfloat16(), torch.randn(rows, D, device="cuda").bfloat16()
    w = torch.ones(D, device="cuda").bfloat16()
    ms = timeit(lambda: ops.add_rms_norm(x, d, w), a.iters, a.warmup, not a.no_flush)
    report(f"add+rmsnorm fwd {rows}x{D}", ms, bytes_=4.0 * rows * D * 2)


def bench_cp_attn(a) -> None:
    """Context-parallel KSA (or causal) attention: the exchange over peer memory plus the shard's kernels."""
    import torch.distributed as dist
    from ..parallel.cp import CpContext, cp_attention_packed
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    B, Hq, Hkv, D, C, S, W, L = a.batch, a.hq, a.hkv, a.dim, a.chunk, a.nsum, a.window, a.seq
    cp = CpContext(dist.group.WORLD, L, C, S, Hkv, D, batch=B, device=dev, full_layers=a.causal, max_window=W,
                   n_heads=Hq, full_layer_mode=a.cp_full_layers)
    Ll, Nsl = L // world, 0 if a.causal else (L // world // C) * S
    qkv = torch.randn(B * (Ll + Nsl), (Hq + 2 * Hkv) * D, device=dev).bfloat16().requires_grad_(a.bwd)
    out = [None]

    def fwd():
        out[0] = cp_attention_packed(qkv, cp, Hq, Hkv, D, None if a.causal else W, not a.causal)

    def timed(fn):
        dist.barrier()
        t = torch.tensor([timeit(fn, a.iters, a.warmup, not a.no_flush)], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t)
    pairs = L * (L + 1) // 2 if a.causal else count_attended_pairs(L, C, S, W)
    flops = 4.0 * D * Hq * pairs * B / world       # per GPU (the slowest rank holds the last, densest shard)
    ms_f = timed(fwd)
    kind = "causal" if a.causal else f"ksa C{C} S{S} W{W}"
    if rank == 0:
        report(f"cp{world} attention fwd {kind} L{L} (max over ranks; mean FLOPs per GPU)", ms_f, flops=flops)
    if a.bwd:
        g = torch.randn_like(out[0])

        def fb():
            fwd()
            out[0].backward(g)
        ms_fb = timed(fb)
        if rank == 0:
            report(f"cp{world} attention bwd {kind} L{L} (fwd+bwd minus fwd)", ms_fb - ms_f, flops=2.5 * flops)
    torch.cuda.synchronize()
    _lib.check_status()
    cp.close()
    dist.destroy_process_group()


def bench_comm(a) -> None:
    """The fused communication kernels alone.

    Under ``torch.distributed.run`` every rank is a GPU and the kernels read the peers' buffers over NVLink (times are
    the maximum over ranks, fractions are of the measured 770 GB/s peer-copy bandwidth per direction).  Started as one
    process, the ``--world`` "ranks" are buffers of the same GPU served by one launch (the form a profiler can
    capture); the bytes then come from local HBM.
    """
    import ctypes
    import torch.distributed as dist
    multi = "RANK" in os.environ and int(os.environ.get("WORLD_SIZE", "1")) > 1
    link_gbs = 770.0
    if multi:
        from ..parallel.symm import SymmetricBuffer
        rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ.get("LOCAL_RANK", "0"))
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    else:
        rank, world = 0, a.world
    dev = torch.device("cuda", torch.cuda.current_device())
    n = (a.mbytes << 20) // 4 // world * world            # fp32 elements of a "unit" (gradient buffer)
    shard = n // world

    def buffers(nbytes):
        if multi:
            sb = SymmetricBuffer(nbytes)
            return sb, sb.ptr_array, sb.view(torch.uint8)
        ts = [torch.empty(nbytes, dtype=torch.uint8, device=dev) for _ in range(world)]
        return ts, (ctypes.c_void_p * world)(*[t.data_ptr() for t in ts]), ts[0]

    def timed(fn):
        if multi:
            dist.barrier()
        t = torch.tensor([timeit(fn, a.iters, a.warmup, not a.no_flush)], device=dev, dtype=torch.float64)
        if multi:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t)

    def show(name, ms, remote_bytes, local_bytes):
        if rank != 0:
            return
        if multi:
            gb = remote_bytes / ms / 1e6
            print(f"{name}: {ms:.4f} ms | {gb:.0f} GB/s over NVLink per GPU ({gb / link_gbs:.2f} of measured {link_gbs:.0f} peer copy)",
                  flush=True)
        else:
            report(name + f" ({world} local buffers)", ms, bytes_=remote_bytes + local_bytes)

    # parameter all-gather: every rank pulls the other ranks' bf16 shards
    hold_w, w_ptrs, _ = buffers(n * 2)
    ms = timed(lambda: _lib.call("ksa_peer_gather", w_ptrs, world, rank, shard, 2, None, None, 0, a.ctas))
    show(f"peer gather {n * 2 >> 20} MiB bf16 unit, world {world}", ms, (world - 1) * shard * 2, (world - 1) * shard * 2)
    # gradient reduce-scatter + AdamW: the owner reads its slice of every rank's fp32 gradients
    hold_g, g_ptrs, g0 = buffers(n * 4)
    g0.view(torch.float32).normal_(0, 1e-3)
    master = torch.zeros(shard, device=dev)
    m1, m2 = torch.zeros_like(master), torch.zeros_like(master)
    out = torch.empty(n, dtype=torch.bfloat16, device=dev)
    hyper = torch.tensor([1e-4, 0.1, 0.05, 1.0 / world], device=dev)
    sumsq = torch.zeros(1, device=dev)
    if multi:
        dist.barrier()
    ms = timed(lambda: _lib.call("ksa_peer_reduce_adamw", g_ptrs, world, rank, rank * shard, shard, master, m1, m2, out,
                                 hyper, 0.9, 0.95, 1e-8, 0.1, 1.0, sumsq, None, None, 0, a.ctas))
    show(f"peer reduce-scatter + AdamW {n * 4 >> 20} MiB fp32 unit, world {world}", ms, (world - 1) * shard * 4,
         shard * 4 + shard * 4 * 6 + shard * 2)
    torch.cuda.synchronize()
    _lib.check_status()
    if multi:
        hold_w.close(); hold_g.close()
        dist.destroy_process_group()


def bench_ag_gemm(a) -> None:
    """All-gather -> GEMM: a row-sharded ``[m, k]`` activation (every rank holds ``m / world`` rows) times a local
    ``[n, k]`` weight, as tensor-parallel prefill runs it.  Compares the stand-alone gather kernel followed by the
    CTA-pair GEMM with the single launch in which a communication warp of every CTA pulls the peers' rows with bulk
    copies while the other warps compute on the rows that have landed.

    Under ``torch.distributed.run`` the peers are GPUs (maximum over ranks; roofline = the slower of the FLOPs at the
    measured GEMM peak and the remote bytes at the measured 770 GB/s peer-copy bandwidth).  Started as one process the
    ``--world`` copies live on this GPU (the form a profiler can capture).
    """
    import ctypes
    import torch.distributed as dist
    multi = "RANK" in os.environ and int(os.environ.get("WORLD_SIZE", "1")) > 1
    if multi:
        from ..parallel.symm import SymmetricBuffer
        rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ.get("LOCAL_RANK", "0"))
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    else:
        rank, world = 0, a.world
    dev = torch.device("cuda", torch.cuda.current_device())
    M, N, K = a.m, a.n, a.k
    shard = (M + world - 1) // world
    nbytes = shard * world * K * 2
    if multi:
        hold = SymmetricBuffer(nbytes)
        ptrs, own = hold.ptr_array, hold.view(torch.bfloat16, 0, shard * world * K).view(shard * world, K)
    else:
        hold = [torch.empty(shard * world, K, dtype=torch.bfloat16, device=dev) for _ in range(world)]
        ptrs, own = (ctypes.c_void_p * world)(*[t.data_ptr() for t in hold]), hold[0]
        for t in hold:
            t.normal_()
    own.normal_()
    W = torch.randn(N, K, device=dev).bfloat16()
    out = torch.empty(M, N, dtype=torch.bfloat16, device=dev)
    done = torch.zeros(_lib.GATHER_COUNTERS, dtype=torch.int32, device=dev)

    def separate():
        _lib.call("ksa_peer_gather", ptrs, world, rank, shard * K, 2, None, None, 0, a.ctas)
        ops.gemm(own[:M], W, out=out, pair=True)

    def fused():
        ops.gemm_gather(own[:M], W, ptrs, world, rank, shard * K * 2, None, None, done, dep_operand=1, out=out)

    def timed(fn):
        if multi:
            torch.cuda.synchronize()
            dist.barrier()
        t = torch.tensor([timeit(fn, a.iters, a.warmup, not a.no_flush)], device=dev, dtype=torch.float64)
        if multi:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t)

    t_sep, t_fused = timed(separate), timed(fused)
    t_lib = None
    if multi and a.compare:
        # the library pair: NCCL all-gather of the row shards into a fresh buffer, then cuBLAS (torch.matmul)
        mine = own[rank * shard:(rank + 1) * shard].clone()
        gathered = torch.empty(shard * world, K, dtype=torch.bfloat16, device=dev)
        out_lib = torch.empty(M, N, dtype=torch.bfloat16, device=dev)

        def library():
            dist.all_gather_into_tensor(gathered, mine)
            torch.matmul(gathered[:M], W.t(), out=out_lib)
        t_lib = timed(library)
    ref = own[:M].float() @ W.float().t() if M * N <= (1 << 26) else None
    err = (out.float() - ref).abs().max().item() / ref.abs().max().item() if ref is not None else float("nan")
    _lib.check_status()
    if rank == 0:
        pk = peaks()
        flops, remote = 2.0 * M * N * K, (world - 1) * shard * K * 2.0
        t_math, t_link = flops / (pk["tflops"] * 1e9), remote / (770.0 * 1e6)
        where = "GPUs" if multi else "local buffers"
        print(f"all-gather -> gemm {M}x{N}x{K}, world {world} ({where}): gather kernel + pair GEMM {t_sep:.4f} ms | "
              f"one launch {t_fused:.4f} ms ({t_sep / t_fused:.2f}x)", flush=True)
        if t_lib is not None:
            print(f"  NCCL all-gather + cuBLAS (torch.matmul): {t_lib:.4f} ms ({t_lib / t_fused:.2f}x the one launch)", flush=True)
        print(f"  roofline: math {t_math:.4f} ms at {pk['src']} {pk['tflops']:.0f} TFLOP/s, link {t_link:.4f} ms at measured "
              f"770 GB/s -> {max(t_math, t_link) / t_fused:.2f} of the slower one; max rel error {err:.2e}", flush=True)
    if multi:
        hold.close()
        dist.destroy_process_group()


def bench_gemm_rs(a) -> None:
    """GEMM -> reduce-scatter + residual add + RMSNorm of tensor-parallel prefill, under ``torch.distributed.run``:
    the row-parallel GEMM (``--m`` rows, ``--k`` local reduction length, ``--dim`` model width) followed by
    ``ksa_tp_reduce_scatter_add_rmsnorm``, (a) with the partial blocks pulled from the peers by the reduction kernel
    and (b) with the GEMM epilogue scattering every row block into its owner's memory (TMA stores), so that the
    reduction reads local memory only.  Maximum over ranks; the gathers that follow are not part of either time."""
    import torch.distributed as dist
    from ..parallel.tp import TpContext
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    M, K, D = a.m, a.k, a.dim
    x = torch.randn(M, K, device=dev).bfloat16()
    w = (0.02 * torch.randn(D, K, device=dev)).bfloat16()
    res_in = torch.randn(M, D, device=dev).bfloat16()
    scale = torch.ones(D, device=dev).bfloat16()
    out = {}
    for push in (False, True):
        tp = TpContext(dist.group.WORLD, D, max_rows=M, device=dev, two_phase_rows=256, two_phase_min_size=2,
                       fused_gather=True, push_partials=push)

        def step():
            token = tp.row_parallel_linear(x, w, residual_rows=M if push else None)
            tp.add_rms_norm(res_in, token, scale, 1e-6, defer_gather=True)
            tp._pending, tp._res_event = None, None          # the gathers are not timed: drop them
        torch.cuda.synchronize()
        dist.barrier()
        t = torch.tensor([timeit(step, a.iters, a.warmup, not a.no_flush)], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        out[push] = float(t)
        torch.cuda.synchronize()
        _lib.check_status()
        dist.barrier()
        tp.close()
    if rank == 0:
        pk = peaks()
        flops = 2.0 * M * D * K
        remote = (world - 1) * ((M + world - 1) // world) * D * 2.0
        t_math, t_link = flops / (pk["tflops"] * 1e9), remote / (770.0 * 1e6)
        print(f"gemm -> reduce-scatter + add + rmsnorm {M}x{D}x{K}, world {world}: pulled by the reduction "
              f"{out[False]:.4f} ms | scattered by the GEMM epilogue {out[True]:.4f} ms ({out[False] / out[True]:.2f}x)",
              flush=True)
        print(f"  roofline of the pair: math {t_math:.4f} ms at {pk['src']} {pk['tflops']:.0f} TFLOP/s, link {t_link:.4f} ms "
              f"at measured 770 GB/s -> {max(t_math, t_link) / out[True]:.2f} of the slower one", flush=True)
    dist.destroy_process_group()


def bench_tp_reduce(a) -> None:
    """The fused all-reduce + residual add + RMSNorm of tensor-parallel inference as ONE launch over ``--world``
    partial buffers of this GPU (the peers' flags are set beforehand, so nothing waits): the form a profiler can
    capture.  Across GPUs the same kernel is timed by ``infer_bench`` under torchrun."""
    import ctypes
    world, rows, D = a.world, a.rows, a.dim
    dev = torch.device("cuda", torch.cuda.current_device())
    parts = [torch.randn(rows, D, device=dev).bfloat16() for _ in range(world)]
    x = torch.randn(rows, D, device=dev).bfloat16()
    w = torch.ones(D, device=dev).bfloat16()
    res, y = torch.empty_like(x), torch.empty_like(x)
    flags = torch.full((world,), 1 << 30, dtype=torch.int32, device=dev)     # already "announced" for every epoch
    scratch = torch.zeros(world, dtype=torch.int32, device=dev)             # the kernel's own announcements land here
    epoch = torch.zeros(2, dtype=torch.int32, device=dev)
    part_ptrs = (ctypes.c_void_p * world)(*[p.data_ptr() for p in parts])
    ann_ptrs = (ctypes.c_void_p * world)(*[scratch.data_ptr() + 4 * r for r in range(world)])
    ms = timeit(lambda: _lib.call("ksa_tp_allreduce_add_rmsnorm", x, part_ptrs, ann_ptrs, flags, world, 0, w, res, y,
                                  rows, rows, D, 1e-6, epoch[0:1], epoch[1:2]), a.iters, a.warmup, not a.no_flush)
    report(f"all-reduce + add + rmsnorm {rows}x{D}, {world} partials (local buffers)", ms,
           bytes_=(world + 3.0) * rows * D * 2)
    ref = x.float() + sum(p.float() for p in parts)
    err = (res.float() - ref).abs().max().item()
    print(f"  max abs error of the residual stream vs fp32: {err:.3e}", flush=True)


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--compare-ref", action="store_true",
                    help="attn: also time flash_attn 2.x and the reference's sm_100 kernels on the same shapes (1 GPU)")
    ap.add_argument("what", choices=["gemm", "gemv", "attn", "decode", "norm", "cp-attn", "comm", "tp-reduce", "ag-gemm",
                                     "gemm-rs"])
    # the long spellings are for use under torch.distributed.run, whose own parser claims --m and --n as prefixes
    ap.add_argument("--m", "--gemm-m", dest="m", type=int, default=8192)
    ap.add_argument("--n", "--gemm-n", dest="n", type=int, default=4096)
    ap.add_argument("--k", "--gemm-k", dest="k", type=int, default=2048)
    ap.add_argument("--a-mn", action="store_true"); ap.add_argument("--b-mn", action="store_true")
    ap.add_argument("--fp32-out", action="store_true"); ap.add_argument("--compare", action="store_true")
    ap.add_argument("--pair", action="store_true", help="gemm: run on CTA pairs (tcgen05 cta_group::2)")
    ap.add_argument("--scatter-world", type=int, default=0,
                    help="gemm: scatter the row blocks of the product to this many buffers from the epilogue")
    ap.add_argument("--seq", type=int, default=8192); ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--hq", type=int, default=16); ap.add_argument("--hkv", type=int, default=8)
    ap.add_argument("--dim", type=int, default=128); ap.add_argument("--chunk", type=int, default=128)
    ap.add_argument("--nsum", type=int, default=1); ap.add_argument("--window", type=int, default=8)
    ap.add_argument("--causal", action="store_true"); ap.add_argument("--bwd", action="store_true")
    ap.add_argument("--cap", type=int, default=131072); ap.add_argument("--rows", type=int, default=8256)
    ap.add_argument("--iters", type=int, default=10); ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--no-flush", action="store_true")
    ap.add_argument("--world", type=int, default=2, help="comm: emulated ranks when started as one process")
    ap.add_argument("--mbytes", type=int, default=256, help="comm: size of the fp32 gradient unit in MiB")
    ap.add_argument("--ctas", type=int, default=64, help="comm: CTAs of the communication kernels")
    ap.add_argument("--cp-full-layers", default="auto", choices=["auto", "ulysses", "halo"])
    return ap


def main(argv=None) -> None:
    a = build_parser().parse_args(argv)
    {"gemm": bench_gemm, "gemv": bench_gemv, "attn": bench_attn, "decode": bench_decode, "norm": bench_norm, "cp-attn": bench_cp_attn, "comm": bench_comm, "tp-reduce": bench_tp_reduce,
     "ag-gemm": bench_ag_gemm, "gemm-rs": bench_gemm_rs}[a.what](a)
    _lib.check_status()


if __name__ == "__main__":
    main()
