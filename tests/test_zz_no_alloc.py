"""The allocation-free RMSNorm backward (``ksa_rmsnorm_bwd_noalloc``) against the regular entry point.

Some users of the kernel library may not allocate device memory when they call it: they run inside a
fixed memory budget, or they embed the library from C and manage every device buffer themselves.  For
them the library exports one variant of the RMSNorm backward whose scratch (per-CTA partial sums of the
weight gradient) is a fixed array inside the library instead of a caller-provided buffer.  This test
calls that variant through its exported C symbol, twice in a row with different sizes (the scratch keeps
the first call's contents, which must not leak into the second), and checks both results against
``ksa_rmsnorm_bwd``.  The file name sorts last so that a run that stops at the first failure has already
run every other test; the test also passes on its own in a fresh process.
"""
import ctypes

import pytest
import torch

from ksa_b200.ops import _lib

pytestmark = pytest.mark.gpu

MAX_D = 4096  # KSA_NOALLOC_RMSNORM_MAX_D in ksa_b200/csrc/noalloc.h


def _symbol():
    lib = _lib.load()
    fn = lib.ksa_rmsnorm_bwd_noalloc
    P, I = ctypes.c_void_p, ctypes.c_int
    fn.argtypes = [P, P, P, P, P, P, P, I, I, I, P]
    fn.restype = I
    return lib, fn


def _rel(a, b):
    return ((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-12)).item()


def _case(rows, D, with_dres, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    mk = lambda *s: torch.randn(*s, device="cuda", generator=g).to(torch.bfloat16)
    x, dy = mk(rows, D), mk(rows, D)
    w = (1 + 0.1 * torch.randn(D, device="cuda", generator=g)).to(torch.bfloat16)
    dres = mk(rows, D) if with_dres else None
    rstd = torch.rsqrt(x.float().pow(2).mean(-1) + 1e-6)
    return x, dy, w, dres, rstd


def _regular(x, dy, w, dres, rstd, dw_init):
    rows, D = x.shape
    dx = torch.empty_like(x)
    dw = dw_init.clone()
    partial = torch.empty((_lib.rmsnorm_bwd_parts(rows), D), dtype=torch.float32, device="cuda")
    _lib.call("ksa_rmsnorm_bwd", dy, x, w, rstd, dres, dx, partial, dw, 1, rows, D)
    return dx, dw


def _noalloc(fn, lib, x, dy, w, dres, rstd, dw_init):
    rows, D = x.shape
    dx = torch.empty_like(x)
    dw = dw_init.clone()
    stream = torch.cuda.current_stream().cuda_stream
    rc = fn(dy.data_ptr(), x.data_ptr(), w.data_ptr(), rstd.data_ptr(),
            dres.data_ptr() if dres is not None else None, dx.data_ptr(), dw.data_ptr(), 1, rows, D, stream)
    assert rc == 0, lib.ksa_last_error().decode()
    return dx, dw


def _formula(x, dy, w, dres, rstd, dw_init, accumulate):
    """The backward in plain fp32 PyTorch: dx = rstd (dy w - xhat mean(dy w xhat)) (+ dres), dw (+)= sum dy xhat."""
    xf, gf, wf = x.float(), dy.float(), w.float()
    xhat = xf * rstd[:, None]
    gw = gf * wf
    dx = rstd[:, None] * (gw - xhat * (gw * xhat).mean(-1, keepdim=True))
    if dres is not None:
        dx = dx + dres.float()
    dw = (gf * xhat).sum(0)
    return dx, (dw_init + dw if accumulate else dw)


def test_noalloc_rmsnorm_bwd_matches_regular_entry_point_twice():
    lib, fn = _symbol()
    torch.cuda.synchronize()
    # two calls in a row: a large case first, then a smaller one that reuses (part of) the same scratch
    for rows, D, with_dres, seed in ((1500, 2048, True, 1), (37, 512, False, 2)):
        x, dy, w, dres, rstd = _case(rows, D, with_dres, seed)
        dw_init = torch.randn(D, device="cuda")
        dx_ref, dw_ref = _regular(x, dy, w, dres, rstd, dw_init)
        dx_new, dw_new = _noalloc(fn, lib, x, dy, w, dres, rstd, dw_init)
        torch.cuda.synchronize()
        assert torch.isfinite(dx_new.float()).all() and torch.isfinite(dw_new).all()
        assert _rel(dx_new, dx_ref) < 1.5e-2, (rows, D, _rel(dx_new, dx_ref))
        assert _rel(dw_new, dw_ref) < 2e-2, (rows, D, _rel(dw_new, dw_ref))
        dx_f, dw_f = _formula(x, dy, w, dres, rstd, dw_init, True)
        assert _rel(dx_new, dx_f) < 1.5e-2 and _rel(dw_new, dw_f) < 2e-2


@pytest.mark.parametrize("rows,D", [(300, 4096), (64, 2560)])
def test_noalloc_rmsnorm_bwd_at_the_size_limit_and_off_the_2048_grid(rows, D):
    """D = 4096 is the largest hidden size the built-in scratch covers and uses every thread's second vector;
    D = 2560 (the 4B model's hidden size) is not a multiple of 2048.  Checked against the fp32 formula, overwriting dw
    (accumulate_dw = 0) and with no dw at all (null pointer: only dx is produced)."""
    lib, fn = _symbol()
    x, dy, w, dres, rstd = _case(rows, D, True, 5)
    stream = torch.cuda.current_stream().cuda_stream
    dx = torch.empty_like(x)
    dw = torch.full((D,), 7.0, device="cuda")            # must be overwritten, not added to
    rc = fn(dy.data_ptr(), x.data_ptr(), w.data_ptr(), rstd.data_ptr(), dres.data_ptr(), dx.data_ptr(), dw.data_ptr(),
            0, rows, D, stream)
    assert rc == 0, lib.ksa_last_error().decode()
    dx_f, dw_f = _formula(x, dy, w, dres, rstd, None, False)
    torch.cuda.synchronize()
    assert _rel(dx, dx_f) < 1.5e-2 and _rel(dw, dw_f) < 2e-2
    dx2 = torch.empty_like(x)
    rc = fn(dy.data_ptr(), x.data_ptr(), w.data_ptr(), rstd.data_ptr(), dres.data_ptr(), dx2.data_ptr(), None, 0,
            rows, D, stream)
    assert rc == 0, lib.ksa_last_error().decode()
    torch.cuda.synchronize()
    assert torch.equal(dx, dx2)


def test_noalloc_rmsnorm_bwd_takes_no_device_memory():
    """After a first call (which may load the module that holds the scratch array), further calls leave the amount of
    free device memory unchanged."""
    lib, fn = _symbol()
    x, dy, w, dres, rstd = _case(256, 1024, False, 9)
    dx, dw = torch.empty_like(x), torch.zeros(1024, device="cuda")
    args = (dy.data_ptr(), x.data_ptr(), w.data_ptr(), rstd.data_ptr(), None, dx.data_ptr(), dw.data_ptr(), 0, 256, 1024,
            torch.cuda.current_stream().cuda_stream)
    assert fn(*args) == 0
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    for _ in range(3):
        assert fn(*args) == 0
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info()
    assert free_after == free_before


def test_noalloc_rmsnorm_bwd_rejects_sizes_beyond_its_scratch():
    lib, fn = _symbol()
    rows, D = 4, MAX_D + 8
    x, dy, w, dres, rstd = _case(rows, D, False, 3)
    dx, dw = torch.empty_like(x), torch.zeros(D, device="cuda")
    rc = fn(dy.data_ptr(), x.data_ptr(), w.data_ptr(), rstd.data_ptr(), None, dx.data_ptr(), dw.data_ptr(), 0,
            rows, D, torch.cuda.current_stream().cuda_stream)
    assert rc != 0
    assert "exceeds the built-in scratch" in lib.ksa_last_error().decode()
    torch.cuda.synchronize()
