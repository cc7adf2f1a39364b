"""The fused context-parallel exchange (``ksa_b200/parallel/cp.py``: symmetric slots, flags, P2P copy kernels, head
resharding) on 2, 4 and 8 ranks without a GPU.

Every rank is a thread with its own ``CpContext``; symmetric buffers are CPU tensors reachable through their
addresses, and the copy / add / flag kernels are Python stand-ins that honour the same pointers, sizes, pitches and
flag values (a copy really waits until the owner's flag has reached the exchange number).  The sharded model's loss,
hidden states and gradients are compared with the whole-sequence model, as in the gloo test of the collective path.
"""
import copy
import threading
import time

import pytest
import torch
import torch.distributed as dist

from ksa_b200 import ops
from ksa_b200.ops import _lib
from ksa_b200.parallel import cp as cp_mod, symm
from ksa_b200.parallel.cp import CpContext, shard_inputs

from test_cp_cpu import _build, _cfg
from test_tp_layout_cpu import FakeSymm, Group, Memory, _ptrs, _run_ranks


class ZeroedSymm(FakeSymm):
    """Symmetric memory comes zeroed (the flags start at 0)."""

    def __init__(self, nbytes, group=None, device=None):
        super().__init__(nbytes, group, device)
        self._bytes.zero_()


def _raw(mem: Memory, ptr: int, nbytes: int) -> torch.Tensor:
    for t in mem.blocks:
        lo = t.data_ptr()
        if lo <= ptr and ptr + nbytes <= lo + t.numel() * t.element_size():
            return t.view(torch.uint8)[ptr - lo:ptr - lo + nbytes]
    raise AssertionError(f"a kernel was pointed at unmapped memory: {ptr:#x} + {nbytes}")


def make_cp_kernels(mem: Memory, log: list):
    lock = threading.Lock()

    def flag(ptr):
        return int(_raw(mem, ptr, 4).view(torch.int32)[0])

    def wait(ptr, target):
        t0 = time.monotonic()
        while flag(ptr) < target:
            if time.monotonic() - t0 > 60:
                raise AssertionError(f"a wait for flag value {target} ran out (flag holds {flag(ptr)})")
            time.sleep(0.0005)

    def value(epoch, add):
        return (int(epoch[0]) if epoch is not None else 0) + add

    def call(name, *a):
        log.append(name)
        if name == "ksa_signal_set":
            ptrs, world, epoch, add = a
            with lock:
                for p in _ptrs(ptrs, world):
                    _raw(mem, p, 4).view(torch.int32)[0] = value(epoch, add)
        elif name == "ksa_signal_wait":
            base, n, epoch, add = a
            for i in range(n):
                wait(base + 4 * i, value(epoch, add))
        elif name == "ksa_peer_copy":
            dst, src, nbytes, flag_ptr, epoch, add, _ctas = a
            wait(flag_ptr, value(epoch, add))
            assert dst.is_contiguous() and dst.numel() * dst.element_size() == nbytes
            dst.view(-1).view(torch.uint8).copy_(_raw(mem, src, nbytes))
        elif name == "ksa_peer_add_bf16":
            dst, src, numel, flag_ptr, epoch, add, _ctas = a
            wait(flag_ptr, value(epoch, add))
            assert dst.is_contiguous() and dst.numel() == numel
            dst.view(-1).add_(_raw(mem, src, numel * dst.element_size()).view(dst.dtype))
        elif name == "ksa_peer_copy2d":
            dst, dpitch, src, spitch, rows, width, flag_ptr, epoch, add, _ctas = a
            wait(flag_ptr, value(epoch, add))
            item = dst.element_size()
            assert dst.shape == (rows, width // item) and dst.stride(0) * item == dpitch
            for i in range(rows):
                dst[i].view(torch.uint8).copy_(_raw(mem, src + i * spitch, width))
        else:
            raise AssertionError(f"unexpected kernel {name}")
    return call


def apply_cp_patches(monkeypatch):
    """Route CpContext's fused path onto the stand-ins (also used by the combined FSDP + context-parallel test)."""
    monkeypatch.setattr(CpContext, "_on_gpus", staticmethod(lambda device: True))
    monkeypatch.setattr(symm, "SymmetricBuffer", ZeroedSymm)
    monkeypatch.setattr(dist, "get_rank", lambda g=None: g.rank)
    monkeypatch.setattr(dist, "get_world_size", lambda g=None: g.size)
    monkeypatch.setattr(torch.cuda, "synchronize", lambda device=None: None)

    # the attention kernels with offsets: the dense-mask shard attention of the collective path stands in for them
    def ksa_attention(q_t, k_t, v_t, q_s, k_s, v_s, chunk, n_sum, window, scale, q_off=0, k_off=0, s_off=0, seq_len=None):
        Ll = q_t.shape[1]
        sh = cp_mod.CpShape(q_off // Ll, seq_len // Ll, seq_len, chunk, n_sum)
        return cp_mod._cpu_shard_attention(q_t, k_t, v_t, q_s, k_s, v_s, sh, q_off - k_off, window, 0, scale)

    def shard_causal_attention(q_t, k_t, v_t, scale, tok_window, q_off=0, k_off=0, seq_len=None):
        Ll = q_t.shape[1]
        sh = cp_mod.CpShape(q_off // Ll, seq_len // Ll, seq_len, 1, 0)
        return cp_mod._cpu_shard_attention(q_t, k_t, v_t, None, None, None, sh, q_off - k_off, None, tok_window, scale)[0]
    monkeypatch.setattr(ops, "ksa_attention", ksa_attention)
    monkeypatch.setattr(ops, "shard_causal_attention", shard_causal_attention)


@pytest.fixture
def fake_cp_gpu(monkeypatch):
    apply_cp_patches(monkeypatch)
    yield


@pytest.mark.parametrize("world,L,chunk,window,n_sum,mode", [(2, 128, 16, 2, 1, "auto"), (4, 128, 16, 3, 2, "halo"),
                                                             (4, 256, 16, 5, 1, "auto"), (8, 256, 16, 3, 1, "halo")])
def test_fused_exchange_matches_whole_sequence(fake_cp_gpu, monkeypatch, world, L, chunk, window, n_sum, mode):
    cfg = _cfg(chunk, window, n_sum)
    if mode == "auto":                                   # head resharding needs the heads to divide by the ranks
        cfg = cfg.merge({"num_heads": 4, "num_kv_heads": 4}) if world == 4 else cfg
    B = 2
    g = torch.Generator().manual_seed(3)
    toks = torch.randint(0, 200, (B, L + 1), generator=g)
    log, results = [], {}
    whole = _build(cfg)                                  # built once: the global random generator is not per thread

    def body(rank, group):
        if rank == 0:
            monkeypatch.setattr(_lib, "call", make_cp_kernels(group.shared["mem"], log))
        group.shared["barrier"].wait()
        model = copy.deepcopy(whole)
        tokens, labels = shard_inputs(toks[:, :-1], toks[:, 1:], rank, world)
        model.cp = CpContext(group, L, chunk, n_sum, cfg.num_kv_heads, cfg.head_dim, batch=B, device="cuda",
                             dtype=torch.float32, n_heads=cfg.num_heads, full_layers=True, max_window=window,
                             full_layer_mode=mode)
        assert model.cp.fused
        losses = []
        for _ in range(2):                               # two steps: every slot is used again
            model.zero_grad()
            loss = model(tokens, labels)
            loss.backward()
            losses.append(float(loss.detach()))
        grads = {n: p.grad.clone() for n, p in model.named_parameters() if p.grad is not None}
        with torch.no_grad():
            hidden = model(tokens, return_hidden=True)
        results[rank] = (losses, grads, hidden, model.cp.full_layer_mode)
        group.shared["barrier"].wait()
        model.cp.close()

    _run_ranks(world, body)
    model = whole
    loss = model(toks[:, :-1].contiguous(), toks[:, 1:].contiguous())
    loss.backward()
    hidden = model(toks[:, :-1].contiguous(), return_hidden=True).detach()
    Ll = L // world
    for step in range(2):
        assert abs(sum(results[r][0][step] for r in range(world)) / world - float(loss.detach())) < 1e-5
    for r in range(world):
        torch.testing.assert_close(results[r][2], hidden[:, r * Ll:(r + 1) * Ll], atol=2e-5, rtol=1e-4)
    for n, p in model.named_parameters():
        if p.grad is None:
            continue
        avg = sum(results[r][1][n] for r in range(world)) / world
        torch.testing.assert_close(avg, p.grad, atol=2e-5, rtol=1e-3, msg=lambda m: f"{n}: {m}")
    assert "ksa_peer_copy" in log and "ksa_peer_add_bf16" in log
    assert ("ksa_peer_copy2d" in log) == (results[0][3] == "ulysses")
