"""The host side of tensor-parallel prefill (``ksa_b200/parallel/tp.py``) on 2, 3 and 4 ranks without a GPU.

Every rank is a thread with its own ``TpContext``; the symmetric buffers are CPU tensors that all threads can reach
through their addresses, and the kernel library is replaced by Python functions that do what the kernels do with the
pointers, sizes and offsets they are given (scatter of row blocks, reduce-scatter + add + RMSNorm over partial
pointers, shard gathers, all-gather -> GEMM).  A barrier inside the stand-ins plays the part of the flags.  What is
checked is the layout arithmetic of the host code: slot offsets, the scattered layout of a slot, the biased partial
pointers, shard sizes, and the hand-over of deferred gathers - against a plain computation over all ranks' data.
"""
import contextlib
import ctypes
import threading

import pytest
import torch
import torch.distributed as dist

from ksa_b200 import ops
from ksa_b200.ops import _lib
from ksa_b200.parallel import symm, tp as tp_mod
from ksa_b200.parallel.tp import TpContext

BF = torch.bfloat16


class Memory:
    """Address -> tensor lookup over everything the stand-in kernels may be pointed at."""

    def __init__(self):
        self.blocks = []
        self.lock = threading.Lock()

    def add(self, t: torch.Tensor) -> torch.Tensor:
        with self.lock:
            self.blocks.append(t)
        return t

    def bf16(self, ptr: int, numel: int) -> torch.Tensor:
        for t in self.blocks:
            lo = t.data_ptr()
            if lo <= ptr and ptr + 2 * numel <= lo + t.numel() * t.element_size():
                return t.view(torch.uint8)[ptr - lo:ptr - lo + 2 * numel].view(BF)
        raise AssertionError(f"a kernel was pointed at unmapped memory: {ptr:#x} + {2 * numel}")


class Group:
    def __init__(self, rank, size, shared):
        self.rank, self.size, self.shared = rank, size, shared


class FakeSymm:
    """Stand-in for SymmetricBuffer: rank r's copy is a CPU tensor; all copies are known to every rank."""

    def __init__(self, nbytes, group, device):
        sh = group.shared
        with sh["lock"]:
            idx = sh["alloc_count"][group.rank]
            sh["alloc_count"][group.rank] += 1
            copies = sh["buffers"].setdefault(idx, {})
            copies[group.rank] = sh["mem"].add(torch.full((nbytes + 64,), 0x7F, dtype=torch.uint8))
        sh["barrier"].wait()
        self.world, self.rank, self.nbytes = group.size, group.rank, nbytes
        self._bytes = copies[group.rank][:nbytes]
        self.peer_ptrs = [copies[r].data_ptr() for r in range(group.size)]
        self.local_ptr = self.peer_ptrs[group.rank]
        self.ptr_array = (ctypes.c_void_p * self.world)(*self.peer_ptrs)

    view = symm.SymmetricBuffer.view
    offset_ptr_array = symm.SymmetricBuffer.offset_ptr_array

    def close(self):
        pass


class FakePad:
    def __init__(self, n, group, device):
        self.flags = torch.zeros(n, dtype=torch.int32)
        self._base = self.flags.data_ptr()
        self.world = group.size

    def flag_ptrs(self, index):
        return (ctypes.c_void_p * self.world)(*[self._base + 4 * index] * self.world)

    def local_ptr(self, index):
        return self._base + 4 * index

    def close(self):
        pass


def _ptrs(arr, n):
    return [int(arr[i]) for i in range(n)]


def make_kernels(mem: Memory, barrier: threading.Barrier, log: list):
    """Python stand-ins for the entry points that ``TpContext`` launches (same argument lists, minus the stream)."""

    def gather(ptrs, world, rank, shard_elems, elem_bytes):
        n = shard_elems * elem_bytes // 2
        barrier.wait()                                        # the owners have written their shards
        for r in range(world):
            if r != rank:
                mem.bf16(ptrs[rank] + 2 * n * r, n).copy_(mem.bf16(ptrs[r] + 2 * n * r, n))

    def reduce_rows(x, partial_ptrs, world, w, res, y, rows_d, D, eps, lo, hi):
        barrier.wait()                                        # every rank's partial block is in place
        for row in range(lo, hi):
            v = x[row].float()
            if row < rows_d:
                acc = torch.zeros(D)
                for r in range(world):
                    acc += mem.bf16(partial_ptrs[r] + 2 * D * row, D).float()
                v = (v + acc).to(BF).float()
            res[row] = v.to(BF)
            y[row] = (v * torch.rsqrt((v * v).mean() + eps) * w.float()).to(BF)

    def call(name, *a):
        log.append(name)
        if name == "ksa_gemm2_scatter_bf16":
            x, w, M, N, K, lda, ldb, ldc, targets, world, shard = a
            prod = (x.float() @ w.float().t()).to(BF)
            for r, base in enumerate(_ptrs(targets, world)):
                lo, hi = min(r * shard, M), min((r + 1) * shard, M)
                if hi > lo:
                    mem.bf16(base, (hi - lo) * ldc).view(hi - lo, ldc)[:, :N].copy_(prod[lo:hi])
        elif name == "ksa_tp_reduce_scatter_add_rmsnorm":
            x, pp, _ann, _fl, world, rank, w, res, y, rows_x, rows_d, D, eps, _e, _d, lo, hi, _notify = a
            reduce_rows(x, _ptrs(pp, world), world, w, res, y, rows_d, D, eps, lo, hi)
        elif name == "ksa_tp_allreduce_add_rmsnorm":
            x, pp, _ann, _fl, world, rank, w, res, y, rows_x, rows_d, D, eps, _e, _d = a
            reduce_rows(x, _ptrs(pp, world), world, w, res, y, rows_d, D, eps, 0, rows_x)
        elif name == "ksa_peer_gather":
            ptrs, world, rank, shard_elems, elem_bytes = a[:5]
            gather(_ptrs(ptrs, world), world, rank, shard_elems, elem_bytes)
        else:
            raise AssertionError(f"unexpected kernel {name}")

    def gemm(x, w, out=None, **kw):
        log.append("gemm")
        r = (x.float() @ w.float().t()).to(BF)
        if out is None:
            return r
        out.copy_(r)
        return out

    def gemm_gather(a, b, peers, world, rank, shard_bytes, ready, epoch, done, *, dep_operand=1, dep_offset=0,
                    epoch_add=0, out=None, out_dtype=BF):
        log.append("gemm_gather")
        assert dep_operand == 1 and a.data_ptr() == int(peers[rank]) + dep_offset
        gather(_ptrs(peers, world), world, rank, shard_bytes, 1)
        return gemm(a, b, out=out)

    return call, gemm, gemm_gather


class _FakeStream:
    def wait_stream(self, other):
        pass

    def wait_event(self, ev):
        pass


class _FakeEvent:
    def record(self, stream=None):
        pass


@pytest.fixture
def fake_gpu(monkeypatch):
    """Route TpContext's fused path onto the stand-ins."""
    monkeypatch.setattr(TpContext, "_on_gpus", staticmethod(lambda device: True))
    monkeypatch.setattr(symm, "SymmetricBuffer", FakeSymm)
    monkeypatch.setattr(symm, "SignalPad", FakePad)
    monkeypatch.setattr(dist, "get_rank", lambda g=None: g.rank)
    monkeypatch.setattr(dist, "get_world_size", lambda g=None: g.size)
    monkeypatch.setattr(dist, "barrier", lambda g=None: g.shared["barrier"].wait())
    monkeypatch.setattr(torch.cuda, "synchronize", lambda device=None: None)
    monkeypatch.setattr(torch.cuda, "Stream", lambda device=None: _FakeStream())
    monkeypatch.setattr(torch.cuda, "current_stream", lambda device=None: _FakeStream())
    monkeypatch.setattr(torch.cuda, "stream", lambda s: contextlib.nullcontext())
    monkeypatch.setattr(torch.cuda, "Event", lambda **kw: _FakeEvent())
    real_zeros = torch.zeros
    monkeypatch.setattr(torch, "zeros", lambda *a, **kw: real_zeros(*a, **{k: v for k, v in kw.items() if k != "device"}))
    yield


def _reference(x, acts, wrs, w, rows_d, eps=1e-6):
    total = sum((a.float() @ wr.float().t()).to(BF).float() for a, wr in zip(acts, wrs))
    v = x.float().clone()
    v[:rows_d] = (v[:rows_d] + total).to(BF).float()
    y = (v * torch.rsqrt((v * v).mean(-1, keepdim=True) + eps) * w.float()).to(BF)
    return v.to(BF), y


def _run_ranks(T, body):
    """Run ``body(rank, group)`` on T threads; re-raise the first failure."""
    shared = {"lock": threading.Lock(), "alloc_count": [0] * T, "buffers": {}, "mem": Memory(),
              "barrier": threading.Barrier(T, timeout=60)}
    errors = []

    def run(rank):
        try:
            body(rank, Group(rank, T, shared))
        except BaseException as e:  # noqa: BLE001 - reported below, the other threads are released
            errors.append(e)
            shared["barrier"].abort()
    threads = [threading.Thread(target=run, args=(r,)) for r in range(T)]
    for t in threads:
        t.start()
    for t in threads:
        t.join(120)
    real = [e for e in errors if not isinstance(e, threading.BrokenBarrierError)]
    if real or errors:
        raise (real or errors)[0]
    return shared


@pytest.mark.parametrize("T", [2, 3, 4])
@pytest.mark.parametrize("push,fused", [(False, False), (False, True), (True, False), (True, True)])
def test_two_phase_layouts_against_a_plain_computation(fake_gpu, monkeypatch, T, push, fused):
    D, Kr, Nc, rows_x, rows_d = 64, 48, 40, 70, 61          # 70 rows do not divide by 3 or 4: ragged last shard
    g = torch.Generator().manual_seed(7)
    x = torch.randn(rows_x, D, generator=g).to(BF)
    w = (1 + 0.1 * torch.randn(D, generator=g)).to(BF)
    wc = (0.1 * torch.randn(Nc, D, generator=g)).to(BF)
    acts = [[torch.randn(rows_d, Kr, generator=g).to(BF) for _ in range(T)] for _ in range(3)]
    wrs = [[(0.1 * torch.randn(D, Kr, generator=g)).to(BF) for _ in range(T)] for _ in range(3)]
    # three chained exchanges: the residual output of one is the input of the next (both slots, a slot reuse)
    refs, cur = [], x
    for k in range(3):
        res, y = _reference(cur, acts[k], wrs[k], w, rows_d)
        refs.append((res, y, (y.float() @ wc.float().t()).to(BF)))
        cur = res
    log = []
    results = {}

    def body(rank, group):
        mem = group.shared["mem"]
        if rank == 0:
            call, gemm, gemm_gather = make_kernels(mem, group.shared["barrier"], log)
            monkeypatch.setattr(_lib, "call", call)
            monkeypatch.setattr(ops, "gemm", gemm)
            monkeypatch.setattr(ops, "gemm_gather", gemm_gather)
        group.shared["barrier"].wait()
        tp = TpContext(group, D, max_rows=rows_x, device="cuda", two_phase_rows=16, two_phase_min_size=2,
                       fused_gather=fused, push_partials=push)
        assert tp.two_phase_rows and tp.fused_gather == fused and tp.push_partials == push
        out, cur = [], x.clone()
        for k in range(3):
            token = tp.row_parallel_linear(acts[k][rank], wrs[k][rank], residual_rows=rows_x)
            res, y = tp.add_rms_norm(cur, token, w, 1e-6, defer_gather=True)
            proj = tp.col_parallel_linear(y, wc)
            tp.flush()
            group.shared["barrier"].wait()           # everybody has read what the next exchange overwrites
            out.append((res.clone(), y.clone(), proj.clone()))
            cur = res
        results[rank] = out
        tp.close()

    _run_ranks(T, body)
    for rank in range(T):
        for k in range(3):
            for got, want, what in zip(results[rank][k], refs[k], ("residual", "normalised", "projection")):
                torch.testing.assert_close(got.float(), want.float(), atol=3e-2, rtol=3e-2,
                                           msg=lambda m: f"rank {rank} exchange {k} {what}: {m}")
    assert ("ksa_gemm2_scatter_bf16" in log) == push
    assert ("gemm_gather" in log) == fused


@pytest.mark.parametrize("T", [2, 4])
def test_few_rows_take_the_one_shot_all_reduce(fake_gpu, monkeypatch, T):
    """Decode-sized calls stay on the one-shot form (every rank sums all partial blocks) whatever the prefill options."""
    D, Kr, rows = 64, 32, 5
    g = torch.Generator().manual_seed(3)
    x = torch.randn(rows, D, generator=g).to(BF)
    w = (1 + 0.1 * torch.randn(D, generator=g)).to(BF)
    acts = [torch.randn(rows, Kr, generator=g).to(BF) for _ in range(T)]
    wrs = [(0.1 * torch.randn(D, Kr, generator=g)).to(BF) for _ in range(T)]
    want_res, want_y = _reference(x, acts, wrs, w, rows)
    log, results = [], {}

    def body(rank, group):
        if rank == 0:
            call, gemm, gemm_gather = make_kernels(group.shared["mem"], group.shared["barrier"], log)
            monkeypatch.setattr(_lib, "call", call)
            monkeypatch.setattr(ops, "gemm", gemm)
            monkeypatch.setattr(ops, "gemm_gather", gemm_gather)
        group.shared["barrier"].wait()
        tp = TpContext(group, D, max_rows=64, device="cuda", two_phase_rows=16, two_phase_min_size=2,
                       fused_gather=True, push_partials=True)
        token = tp.row_parallel_linear(acts[rank], wrs[rank], residual_rows=rows)
        res, y = tp.add_rms_norm(x, token, w, 1e-6, defer_gather=True)
        results[rank] = (res.clone(), y.clone())
        group.shared["barrier"].wait()
        tp.close()

    _run_ranks(T, body)
    for rank in range(T):
        torch.testing.assert_close(results[rank][0].float(), want_res.float(), atol=3e-2, rtol=3e-2)
        torch.testing.assert_close(results[rank][1].float(), want_y.float(), atol=3e-2, rtol=3e-2)
    assert "ksa_tp_allreduce_add_rmsnorm" in log and "ksa_gemm2_scatter_bf16" not in log and "gemm_gather" not in log


@pytest.mark.parametrize("T", [2, 4, 8])
def test_sharded_model_prefill_matches_the_whole_model(fake_gpu, monkeypatch, T):
    """The model's tensor-parallel wiring (deferred gathers, scattered row-parallel outputs, the last layer's
    exception, the flush before the head) on 2, 4 and 8 ranks against the unsharded model, logits of a whole prompt."""
    from ksa_b200.config import get_preset
    from ksa_b200.models import get_model_class
    from ksa_b200.parallel.tp import build_tp_model
    heads = max(4, T)
    cfg = get_preset("qwen3-ksa-tiny").merge({"num_heads": heads, "num_kv_heads": heads, "head_dim": 128 // heads, "embed_dim": 128,
                                              "intermediate_dim": 256, "num_layers": 3, "vocab_size": 512,
                                              "summary_layer_freq": [1, 0, 1], "summary_chunk_size": 32,
                                              "summary_sliding_chunk_num": 2, "summary_token_begin": 512})
    torch.manual_seed(0)
    full = get_model_class(cfg.model_class)(cfg)
    full.init_weights(seed=0)
    full = full.to(BF).eval()
    tokens = torch.randint(0, cfg.vocab_size, (1, 96), generator=torch.Generator().manual_seed(5))
    with torch.no_grad():
        want = full(tokens).float()
    state = {k: v.clone() for k, v in full.state_dict().items()}
    log, results = [], {}

    def all_gather(parts, local, group=None):
        sh = group.shared
        sh.setdefault("ag", {})[group.rank] = local.clone()
        sh["barrier"].wait()
        for r in range(group.size):
            parts[r].copy_(sh["ag"][r])
        sh["barrier"].wait()
    monkeypatch.setattr(dist, "all_gather", all_gather)

    def body(rank, group):
        if rank == 0:
            call, gemm, gemm_gather = make_kernels(group.shared["mem"], group.shared["barrier"], log)
            monkeypatch.setattr(_lib, "call", call)
            monkeypatch.setattr(ops, "gemm", gemm)
            monkeypatch.setattr(ops, "gemm_gather", gemm_gather)
        group.shared["barrier"].wait()
        rows = 96 + 3
        tp = TpContext(group, cfg.embed_dim, max_rows=rows, device="cuda", two_phase_rows=32, two_phase_min_size=2,
                       fused_gather=True, push_partials=True)
        model = build_tp_model(state, cfg, tp, dtype=BF).eval()
        with torch.no_grad():
            results[rank] = model(tokens).float()
        group.shared["barrier"].wait()
        tp.close()

    _run_ranks(T, body)
    for rank in range(T):
        err = (results[rank] - want).abs().max() / want.abs().max()
        assert err < 5e-2, (rank, float(err))
        assert torch.equal(results[rank], results[0]), "the ranks disagree about the logits"
    assert "ksa_gemm2_scatter_bf16" in log and "gemm_gather" in log and "ksa_tp_reduce_scatter_add_rmsnorm" in log


def test_sharded_engine_prefill_and_decode_on_four_ranks(fake_gpu, monkeypatch):
    """Prefill (two-phase form with both fused paths) and a few decode steps (one-shot all-reduce) of the inference
    engine on 4 emulated ranks against the unsharded engine, fed with the same tokens."""
    from ksa_b200.config import get_preset
    from ksa_b200.inference.engine import KsaInferenceEngine
    from ksa_b200.models import get_model_class
    from ksa_b200.parallel.tp import build_tp_model
    T = 4
    cfg = get_preset("qwen3-ksa-tiny").merge({"num_heads": 4, "num_kv_heads": 4, "head_dim": 32, "embed_dim": 128,
                                              "intermediate_dim": 256, "num_layers": 2, "vocab_size": 512,
                                              "summary_layer_freq": [1, 0], "summary_chunk_size": 32,
                                              "summary_sliding_chunk_num": 2, "summary_token_begin": 512})
    torch.manual_seed(0)
    full = get_model_class(cfg.model_class)(cfg)
    full.init_weights(seed=0)
    full = full.to(BF).eval()
    prompt = torch.randint(0, cfg.vocab_size, (2, 80), generator=torch.Generator().manual_seed(9))
    steps = 3

    def run(model, feed=None):
        eng = KsaInferenceEngine(model, max_len=256, batch=2)
        outs = [eng.prefill(prompt)]
        toks = [feed[0] if feed else outs[0].argmax(-1)]
        for _ in range(steps):
            outs.append(eng.decode_step(toks[-1]))
            toks.append(feed[len(toks)] if feed else outs[-1].argmax(-1))
        return torch.stack([o.float() for o in outs]), toks
    want, toks = run(full)
    state = {k: v.clone() for k, v in full.state_dict().items()}
    log, results = [], {}

    def all_gather(parts, local, group=None):
        sh = group.shared
        sh.setdefault("ag", {})[group.rank] = local.clone()
        sh["barrier"].wait()
        for r in range(group.size):
            parts[r].copy_(sh["ag"][r])
        sh["barrier"].wait()
    monkeypatch.setattr(dist, "all_gather", all_gather)

    def body(rank, group):
        if rank == 0:
            call, gemm, gemm_gather = make_kernels(group.shared["mem"], group.shared["barrier"], log)
            monkeypatch.setattr(_lib, "call", call)
            monkeypatch.setattr(ops, "gemm", gemm)
            monkeypatch.setattr(ops, "gemm_gather", gemm_gather)
        group.shared["barrier"].wait()
        tp = TpContext(group, cfg.embed_dim, max_rows=2 * (80 + 3), device="cuda", two_phase_rows=32,
                       two_phase_min_size=2, fused_gather=True, push_partials=True)
        model = build_tp_model(state, cfg, tp, dtype=BF).eval()
        results[rank] = run(model, feed=toks)[0]
        group.shared["barrier"].wait()
        tp.close()

    _run_ranks(T, body)
    for rank in range(T):
        err = (results[rank] - want).abs().max() / want.abs().max()
        assert err < 6e-2, (rank, float(err))
    assert "ksa_gemm2_scatter_bf16" in log and "gemm_gather" in log and "ksa_tp_allreduce_add_rmsnorm" in log


@pytest.mark.parametrize("seed", range(10))
def test_two_phase_layouts_random_shapes(fake_gpu, monkeypatch, seed):
    """Random group sizes and row counts (fewer partial rows than residual rows, shards that end past the last row,
    ranks without any row of their own) with both fused paths on."""
    import random
    rnd = random.Random(seed)
    T = rnd.choice([2, 3, 4, 5, 8])
    rows_x = rnd.randint(16, 140)
    rows_d = rnd.randint(max(1, rows_x - 20), rows_x)
    D, Kr, Nc = 32, 24, 16
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(rows_x, D, generator=g).to(BF)
    w = (1 + 0.1 * torch.randn(D, generator=g)).to(BF)
    wc = (0.1 * torch.randn(Nc, D, generator=g)).to(BF)
    acts = [torch.randn(rows_d, Kr, generator=g).to(BF) for _ in range(T)]
    wrs = [(0.1 * torch.randn(D, Kr, generator=g)).to(BF) for _ in range(T)]
    res_ref, y_ref = _reference(x, acts, wrs, w, rows_d)
    proj_ref = (y_ref.float() @ wc.float().t()).to(BF)
    log, results = [], {}

    def body(rank, group):
        if rank == 0:
            call, gemm, gemm_gather = make_kernels(group.shared["mem"], group.shared["barrier"], log)
            monkeypatch.setattr(_lib, "call", call)
            monkeypatch.setattr(ops, "gemm", gemm)
            monkeypatch.setattr(ops, "gemm_gather", gemm_gather)
        group.shared["barrier"].wait()
        tp = TpContext(group, D, max_rows=rows_x, device="cuda", two_phase_rows=16, two_phase_min_size=2,
                       fused_gather=True, push_partials=True)
        token = tp.row_parallel_linear(acts[rank], wrs[rank], residual_rows=rows_x)
        res, y = tp.add_rms_norm(x, token, w, 1e-6, defer_gather=True)
        proj = tp.col_parallel_linear(y, wc)
        tp.flush()
        group.shared["barrier"].wait()
        results[rank] = (res.clone(), y.clone(), proj.clone())
        tp.close()

    _run_ranks(T, body)
    for rank in range(T):
        for got, want, what in zip(results[rank], (res_ref, y_ref, proj_ref), ("residual", "normalised", "projection")):
            torch.testing.assert_close(got.float(), want.float(), atol=3e-2, rtol=3e-2,
                                       msg=lambda m: f"T={T} rows {rows_x}/{rows_d} rank {rank} {what}: {m}")


@pytest.mark.parametrize("T,push,fused,broken", [(2, True, True, None), (3, False, True, None), (4, True, False, None),
                                                 (2, True, True, "wait_event"), (3, False, True, "wait_stream")])
def test_deferred_gather_schedule_orders_every_conflicting_access(fake_gpu, monkeypatch, T, push, fused, broken):
    """The host-side stream model over the two-phase exchange with deferred gathers: the residual rows are gathered on
    a side stream while the projection that consumes the normalised rows runs, and ``flush`` joins them.  Every
    rank records the accesses of its kernels to its own buffers; no conflicting pair on different streams may be left
    without an event between them, and taking an ordering away (``broken``) must be reported."""
    from ksa_b200.utils import stream_model
    from ksa_b200.utils.stream_model import SimulatedCuda
    sim = SimulatedCuda(per_thread=True)
    sim.install(monkeypatch)                      # over the fixture's do-nothing streams
    if broken:
        monkeypatch.setattr(stream_model._Stream, broken, lambda self, other: None)
    D, Kr, Nc, rows_x, rows_d = 64, 48, 40, 70, 61
    g = torch.Generator().manual_seed(7)
    x = torch.randn(rows_x, D, generator=g).to(BF)
    w = (1 + 0.1 * torch.randn(D, generator=g)).to(BF)
    wc = (0.1 * torch.randn(Nc, D, generator=g)).to(BF)
    acts = [[torch.randn(rows_d, Kr, generator=g).to(BF) for _ in range(T)] for _ in range(3)]
    wrs = [[(0.1 * torch.randn(D, Kr, generator=g)).to(BF) for _ in range(T)] for _ in range(3)]
    log, results = [], {}

    def logging_kernels(mem, barrier):
        call, gemm, gemm_gather = make_kernels(mem, barrier, log)

        def lcall(name, *a):
            tr = sim.trace
            if name in ("ksa_tp_reduce_scatter_add_rmsnorm", "ksa_tp_allreduce_add_rmsnorm"):
                xin, res, y, rows = a[0], a[7], a[8], a[9]
                lo, hi = (a[15], a[16]) if name == "ksa_tp_reduce_scatter_add_rmsnorm" else (0, rows)
                tr.access("reduce + norm kernel", reads=[xin], writes=[res[lo:hi], y[lo:hi]])
            elif name == "ksa_gemm2_scatter_bf16":
                tr.access("row-parallel GEMM with scatter epilogue", reads=[a[0], a[1]])
            return call(name, *a)               # the gather's copies are recorded as they happen

        def lgemm(xin, wt, out=None, **kw):
            sim.trace.access("GEMM", reads=[xin, wt], writes=[out] if out is not None else [])
            return gemm(xin, wt, out=out, **kw)

        def lgemm_gather(a, b, *rest, **kw):
            r = gemm_gather(a, b, *rest, **kw)     # gathers the other ranks' rows of `a` (recorded), then multiplies
            sim.trace.access("GEMM after its gather", reads=[a, b])
            return r
        return lcall, lgemm, lgemm_gather

    def body(rank, group):
        tr = sim.enter_thread()
        mem = group.shared["mem"]
        if rank == 0:
            call, gemm, gemm_gather = logging_kernels(mem, group.shared["barrier"])
            monkeypatch.setattr(_lib, "call", call)
            monkeypatch.setattr(ops, "gemm", gemm)
            monkeypatch.setattr(ops, "gemm_gather", gemm_gather)
        group.shared["barrier"].wait()
        with sim.log_copies():
            tp = TpContext(group, D, max_rows=rows_x, device="cuda", two_phase_rows=16, two_phase_min_size=2,
                           fused_gather=fused, push_partials=push)
            cur = x.clone()
            for k in range(3):
                token = tp.row_parallel_linear(acts[k][rank], wrs[k][rank], residual_rows=rows_x)
                res, y = tp.add_rms_norm(cur, token, w, 1e-6, defer_gather=True)
                proj = tp.col_parallel_linear(y, wc)
                tp.flush()
                tr.access("the layer reads its inputs", reads=[res, y, proj])
                group.shared["barrier"].wait()
                cur = res
            results[rank] = (tr.hazards(), sorted({o.stream for o in tr.ops}))
            tp.close()

    _run_ranks(T, body)
    for rank in range(T):
        hazards, streams = results[rank]
        if broken and fused:
            assert hazards, (rank, broken)
        elif not broken:
            assert hazards == [], (rank, hazards[:4])
        assert (len(streams) >= 2) == fused, streams       # the side stream carries work only with deferred gathers
