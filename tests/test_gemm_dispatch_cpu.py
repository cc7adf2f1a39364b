"""Host-side dispatch of ``ops.gemm``: which entry point a GEMM goes to, and how a parameter all-gather that waits for
a GEMM is attached to it (operand inside the gathered buffer or not, flush).  The kernel
library is replaced by a recorder, so this runs without a GPU."""
import ctypes

import pytest
import torch

from ksa_b200 import ops
from ksa_b200.ops import _lib


@pytest.fixture
def calls(monkeypatch):
    rec = []
    monkeypatch.setattr(_lib, "call", lambda name, *args: rec.append((name, args)))
    monkeypatch.setattr(ops, "_cuda", lambda *t: True, raising=False)
    _lib.take_pair_gather()
    yield rec
    _lib.take_pair_gather()


def _job(buf: torch.Tensor, world=4, rank=1, min_flops=0.0):
    nbytes = buf.numel() * buf.element_size()
    return {"peers": (ctypes.c_void_p * world)(), "world": world, "rank": rank, "shard_bytes": nbytes // world,
            "ready": 0, "epoch": None, "epoch_add": 0, "done": None, "base": buf.data_ptr(),
            "nbytes": nbytes, "min_flops": min_flops}


def test_pending_gather_rides_in_the_first_suitable_gemm(calls):
    unit = torch.zeros(4 * 64 * 256 + 512, dtype=torch.bfloat16)          # a flat "unit": weight at element 512
    w = unit[512:512 + 64 * 256].view(64, 256)
    x = torch.zeros(128, 256, dtype=torch.bfloat16)
    job = _job(unit)
    _lib.attach_pair_gather(job)
    # an MN-major GEMM cannot carry it and leaves it pending
    ops.gemm(x.t().contiguous(), w, a_mn_major=True, out=torch.empty(128, 64, dtype=torch.bfloat16))
    assert calls[-1][0] in ("ksa_gemm_bf16", "ksa_gemm2_bf16") and _lib.pair_gather_pending()
    ops.gemm(x, w, out=torch.empty(128, 64, dtype=torch.bfloat16))
    name, args = calls[-1]
    assert name == "ksa_gemm2_gather_bf16" and not _lib.pair_gather_pending()
    # ..., done, dep_operand, dep_offset
    assert args[-2] == 2 and args[-1] == 512 * 2
    # the next GEMM is a plain one again
    ops.gemm(x, w, out=torch.empty(128, 64, dtype=torch.bfloat16))
    assert calls[-1][0] in ("ksa_gemm_bf16", "ksa_gemm2_bf16")


def test_gather_of_another_buffer_only_shares_the_launch(calls):
    unit = torch.zeros(4096, dtype=torch.bfloat16)
    w = torch.zeros(64, 256, dtype=torch.bfloat16)
    x = torch.zeros(128, 256, dtype=torch.bfloat16)
    _lib.attach_pair_gather(_job(unit))
    ops.gemm(x, w, out=torch.empty(128, 64, dtype=torch.bfloat16))
    name, args = calls[-1]
    assert name == "ksa_gemm2_gather_bf16" and args[-2] == 0 and args[-1] == 0


def test_short_gemms_do_not_take_the_gather_and_flush_runs_it_alone(calls):
    unit = torch.zeros(4096, dtype=torch.bfloat16)
    w = torch.zeros(64, 256, dtype=torch.bfloat16)
    x = torch.zeros(128, 256, dtype=torch.bfloat16)
    job = _job(unit, min_flops=1e12)
    _lib.attach_pair_gather(job)
    ops.gemm(x, w, out=torch.empty(128, 64, dtype=torch.bfloat16))
    assert calls[-1][0] != "ksa_gemm2_gather_bf16" and _lib.pair_gather_pending()
    _lib.flush_pair_gather()
    name, args = calls[-1]
    assert name == "ksa_peer_gather" and args[1:5] == (4, 1, job["shard_bytes"], 1) and not _lib.pair_gather_pending()
    # attaching a second job while one is pending runs the first one alone
    _lib.attach_pair_gather(_job(unit))
    n = len(calls)
    _lib.attach_pair_gather(_job(unit))
    assert len(calls) == n + 1 and calls[-1][0] == "ksa_peer_gather"
