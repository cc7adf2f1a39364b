"""Functional ops of the framework.

Every op has two implementations behind one signature:

* CUDA tensors run the hand-written sm_100a kernels of ``ksa_b200/csrc`` through
  ``torch.autograd.Function`` wrappers (forward and backward are both kernels);
* CPU tensors run the plain PyTorch formulas of :mod:`ksa_b200.ops.reference`,
  which are also the numerics oracle of the GPU tests.

There is no third path: a CUDA tensor never falls back to ATen, and a missing
kernel library on a GPU machine raises.

Weight gradients.  When a weight tensor carries a ``main_grad`` attribute (an
fp32 buffer owned by the training engine), backward kernels write or accumulate
the weight gradient straight into it and autograd sees ``None`` for that input;
``_grad_written`` on the weight tells whether the buffer already holds a
contribution of the current accumulation window.  Otherwise the gradient is
returned to autograd in the weight's dtype.
"""
from __future__ import annotations

import math
import os
from typing import Optional, Tuple

import torch

from . import reference as ref
from . import _lib
from .layout import SummaryLayout, get_layout

UNBOUNDED_WINDOW = 1 << 30
# GEMMs with at least this many 256 x 256 tiles run on CTA pairs (tcgen05 cta_group::2, csrc/gemm2.cu; 74 pairs per
# GPU); below that the single-CTA kernel with 128-row tiles has more CTAs to spread.  0 disables the pair kernel.
GEMM_PAIR_MIN_TILES = int(__import__("os").environ.get("KSA_GEMM_PAIR_MIN_TILES", "32"))


def _cuda(x: torch.Tensor) -> bool:
    return x.is_cuda


def _require_bf16(*ts):
    for t in ts:
        if t is not None and t.dtype != torch.bfloat16:
            raise TypeError(f"the sm_100a kernels take bf16 activations/weights, got {t.dtype}")


# =============================================================================== GEMM
def gemm(a: torch.Tensor, b: torch.Tensor, *, a_mn_major: bool = False, b_mn_major: bool = False,
         out: Optional[torch.Tensor] = None, out_dtype: torch.dtype = torch.bfloat16,
         accumulate: bool = False, alpha: float = 1.0, sm_limit: int = 0,
         pair: Optional[bool] = None) -> torch.Tensor:
    """``C[M,N] = alpha * op(A) op(B) (+ C)`` on the tcgen05 GEMM.

    ``a`` is ``[M,K]`` (or ``[K,M]`` when ``a_mn_major``); ``b`` is ``[N,K]`` (or
    ``[K,N]`` when ``b_mn_major``).  Row strides may exceed the row length
    (views of packed buffers); the last dimension must be contiguous.
    """
    _require_bf16(a, b)
    assert a.dim() == 2 and b.dim() == 2 and a.stride(1) == 1 and b.stride(1) == 1
    M, K = (a.shape[1], a.shape[0]) if a_mn_major else (a.shape[0], a.shape[1])
    N, Kb = (b.shape[1], b.shape[0]) if b_mn_major else (b.shape[0], b.shape[1])
    assert K == Kb, f"reduction mismatch {K} vs {Kb}"
    if out is None:
        out = torch.empty((M, N), dtype=out_dtype, device=a.device)
    assert out.shape == (M, N) and out.stride(1) == 1
    if _lib.pair_gather_pending():
        # a parameter all-gather waits for a GEMM that can carry it: CTA pairs, both operands K-major, bf16 output,
        # long enough to hide the transfer.  Whoever attached it flushes it if no such GEMM comes by.
        if (not a_mn_major and not b_mn_major and out.dtype == torch.bfloat16 and not accumulate and alpha == 1.0
                and sm_limit == 0 and M > 16
                and 2.0 * M * N * K >= _lib.peek_pair_gather().get("min_flops", 0.0)):
            job = _lib.take_pair_gather()
            # does the weight operand live in the buffer that is being gathered?  Then its tiles wait for their shards.
            inside = job["base"] <= b.data_ptr() < job["base"] + job["nbytes"]
            _lib.call("ksa_gemm2_gather_bf16", a, b, out, M, N, K, a.stride(0), b.stride(0), out.stride(0), 0, 0, 1.0,
                      job["peers"], job["world"], job["rank"], job["shard_bytes"], job["ready"], job["epoch"],
                      job["epoch_add"], job["done"], 2 if inside else 0, b.data_ptr() - job["base"] if inside else 0)
            return out
    if (M <= 16 and not a_mn_major and not b_mn_major and out.dtype == torch.bfloat16 and not accumulate
            and alpha == 1.0 and K % 8 == 0):
        # decoding: a few activation rows against a whole weight matrix is a stream of the weights, served by the
        # bandwidth-shaped kernel instead of 128-row tensor-core tiles
        _lib.call("ksa_gemv_bf16", a, b, out, M, N, K, a.stride(0), b.stride(0), out.stride(0))
        return out
    if pair is None:
        pair = (GEMM_PAIR_MIN_TILES > 0 and sm_limit == 0
                and ((M + 255) // 256) * ((N + 255) // 256) >= GEMM_PAIR_MIN_TILES)
    if pair:
        _lib.call("ksa_gemm2_bf16", a, b, out, M, N, K, a.stride(0), b.stride(0), out.stride(0),
                  int(a_mn_major), int(b_mn_major), int(out.dtype == torch.float32), int(accumulate), float(alpha))
        return out
    _lib.call("ksa_gemm_bf16", a, b, out, M, N, K, a.stride(0), b.stride(0), out.stride(0),
              int(a_mn_major), int(b_mn_major), int(out.dtype == torch.float32), int(accumulate),
              float(alpha), int(sm_limit))
    return out


def gemm_gather(a: torch.Tensor, b: torch.Tensor, peers, world: int, rank: int, shard_bytes: int, ready_flags,
                epoch: Optional[torch.Tensor], done: Optional[torch.Tensor], *, dep_operand: int = 1,
                dep_offset: int = 0, epoch_add: int = 0, out: Optional[torch.Tensor] = None,
                out_dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    """All-gather -> GEMM in one launch: ``C = A B^T`` (both K-major) on CTA pairs while a communication warp in
    every CTA of the same launch pulls the other ranks' shards of the gathered buffer over NVLink.

    ``peers``: ctypes array of every rank's pointer to the buffer (``peers[rank]`` is this rank's copy, which the
    gather completes); shard ``r`` is bytes ``[r*shard_bytes, (r+1)*shard_bytes)``.  ``dep_operand`` 1 (2) says that
    ``a`` (``b``) lies in this rank's copy at byte ``dep_offset``: its tiles are read only once the part of the shard
    that holds them has landed.  ``done``: int32 device tensor of ``_lib.GATHER_COUNTERS`` scratch counters (zeroed
    by the call).
    """
    _require_bf16(a, b)
    assert a.dim() == 2 and b.dim() == 2 and a.stride(1) == 1 and b.stride(1) == 1 and a.shape[1] == b.shape[1]
    assert done is None or done.numel() >= _lib.GATHER_COUNTERS
    M, K = a.shape
    N = b.shape[0]
    if out is None:
        out = torch.empty((M, N), dtype=out_dtype, device=a.device)
    assert out.shape == (M, N) and out.stride(1) == 1
    _lib.call("ksa_gemm2_gather_bf16", a, b, out, M, N, K, a.stride(0), b.stride(0), out.stride(0),
              int(out.dtype == torch.float32), 0, 1.0, peers, world, rank, shard_bytes, ready_flags, epoch, epoch_add,
              done, dep_operand, dep_offset)
    return out


def _weight_grad(weight: torch.Tensor, compute):
    """Route a weight gradient: into ``weight.main_grad`` (fp32) or back to autograd.

    ``compute(out, accumulate)`` must fill ``out``; with ``out=None`` it returns a new bf16 tensor.
    """
    mg = getattr(weight, "main_grad", None)
    if mg is not None:
        first = not getattr(weight, "_grad_written", False)
        compute(mg, not first)
        weight._grad_written = True
        return None
    return compute(None, False)


class _LinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight):
        x2 = x.reshape(-1, x.shape[-1])
        if x2.stride(1) != 1:
            x2 = x2.contiguous()
        y = gemm(x2, weight)
        ctx.save_for_backward(x2, weight)
        ctx.x_shape = x.shape
        return y.view(*x.shape[:-1], weight.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x2, weight = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1])
        if dy2.stride(1) != 1:
            dy2 = dy2.contiguous()
        dx = dw = None
        if ctx.needs_input_grad[0]:
            dx = gemm(dy2, weight, b_mn_major=True).view(ctx.x_shape)
        if ctx.needs_input_grad[1]:
            def compute(out, acc):
                if out is None:
                    return gemm(dy2, x2, a_mn_major=True, b_mn_major=True)
                gemm(dy2, x2, a_mn_major=True, b_mn_major=True, out=out, accumulate=acc)
            dw = _weight_grad(weight, compute)
        return dx, dw


def linear(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``x @ weight.T (+ bias)``; the CUDA path is the tcgen05 GEMM for forward, dX and dW."""
    if not _cuda(x):
        return ref.linear(x, weight, bias)
    _require_bf16(x, weight)
    y = _LinearFn.apply(x, weight)
    return y if bias is None else y + bias


class _DualLinearFn(torch.autograd.Function):
    """Rows ``[:n_a]`` use ``w_a``, rows ``[n_a:]`` use ``w_b``; one output buffer, two GEMM launches."""

    @staticmethod
    def forward(ctx, x, w_a, w_b, n_a):
        R = x.shape[0]
        y = torch.empty((R, w_a.shape[0]), dtype=x.dtype, device=x.device)
        if n_a > 0:
            gemm(x[:n_a], w_a, out=y[:n_a])
        if R > n_a:
            gemm(x[n_a:], w_b, out=y[n_a:])
        ctx.save_for_backward(x, w_a, w_b)
        ctx.n_a = n_a
        return y

    @staticmethod
    def backward(ctx, dy):
        x, w_a, w_b = ctx.saved_tensors
        n_a, R = ctx.n_a, x.shape[0]
        dy = dy if dy.is_contiguous() else dy.contiguous()
        dx = None
        if ctx.needs_input_grad[0]:
            dx = torch.empty_like(x)
            if n_a > 0:
                gemm(dy[:n_a], w_a, b_mn_major=True, out=dx[:n_a])
            if R > n_a:
                gemm(dy[n_a:], w_b, b_mn_major=True, out=dx[n_a:])
        grads = []
        for need, w, lo, hi in ((ctx.needs_input_grad[1], w_a, 0, n_a), (ctx.needs_input_grad[2], w_b, n_a, R)):
            if not need or hi <= lo:
                grads.append(None)
                continue
            dys, xs = dy[lo:hi], x[lo:hi]

            def compute(out, acc, dys=dys, xs=xs):
                if out is None:
                    return gemm(dys, xs, a_mn_major=True, b_mn_major=True)
                gemm(dys, xs, a_mn_major=True, b_mn_major=True, out=out, accumulate=acc)
            grads.append(_weight_grad(w, compute))
        return dx, grads[0], grads[1], None


def dual_linear(x: torch.Tensor, w_a: torch.Tensor, w_b: torch.Tensor, n_a: int) -> torch.Tensor:
    """``cat(x[:n_a] @ w_a.T, x[n_a:] @ w_b.T)`` without the concatenation (text rows | summary rows)."""
    if not _cuda(x):
        return torch.cat([ref.linear(x[:n_a], w_a), ref.linear(x[n_a:], w_b)], dim=0)
    _require_bf16(x, w_a, w_b)
    x = x if x.is_contiguous() else x.contiguous()
    return _DualLinearFn.apply(x, w_a, w_b, n_a)


# =============================================================================== RMSNorm
def _rmsnorm_backward(res, weight, rstd, dy, dres, shape):
    rows, D = res.shape
    dy2 = dy.reshape(-1, D)
    dy2 = dy2 if dy2.is_contiguous() else dy2.contiguous()
    dres2 = None
    if dres is not None:
        dres2 = dres.reshape(-1, D)
        dres2 = dres2 if dres2.is_contiguous() else dres2.contiguous()
    dx = torch.empty_like(res)
    parts = _lib.rmsnorm_bwd_parts(rows)
    partial = torch.empty((parts, D), dtype=torch.float32, device=res.device)

    def compute(out, acc):
        if out is None:
            dwf = torch.empty(D, dtype=torch.float32, device=res.device)
            _lib.call("ksa_rmsnorm_bwd", dy2, res, weight, rstd, dres2, dx, partial, dwf, 0, rows, D)
            return dwf.to(weight.dtype)
        _lib.call("ksa_rmsnorm_bwd", dy2, res, weight, rstd, dres2, dx, partial, out, int(acc), rows, D)

    dw = _weight_grad(weight, compute)
    return dx.view(shape), dw


class _AddRmsNormFn(torch.autograd.Function):
    """(x, delta) -> (x + delta, norm(x + delta))."""

    @staticmethod
    def forward(ctx, x, delta, weight, eps):
        D = x.shape[-1]
        x2 = x.reshape(-1, D)
        rows = x2.shape[0]
        y = torch.empty_like(x2)
        res = torch.empty_like(x2)
        rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
        d2 = delta.reshape(-1, D)
        _lib.call("ksa_rmsnorm_fwd", x2, d2, weight, res, y, rstd, rows, D, float(eps), d2.shape[0])
        ctx.save_for_backward(res, weight, rstd)
        ctx.shape = x.shape
        ctx.delta_shape = delta.shape
        return res.view(x.shape), y.view(x.shape)

    @staticmethod
    def backward(ctx, dres, dy):
        res, weight, rstd = ctx.saved_tensors
        if dy is None:
            dy = torch.zeros_like(res)
        dx, dw = _rmsnorm_backward(res, weight, rstd, dy, dres, ctx.shape)
        n_delta = 1
        for d in ctx.delta_shape[:-1]:
            n_delta *= d
        ddelta = dx.reshape(-1, dx.shape[-1])[:n_delta].view(ctx.delta_shape)
        return dx, ddelta, dw, None


class _RmsNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, eps):
        D = x.shape[-1]
        x2 = x.reshape(-1, D)
        rows = x2.shape[0]
        y = torch.empty_like(x2)
        rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
        _lib.call("ksa_rmsnorm_fwd", x2, None, weight, None, y, rstd, rows, D, float(eps), 0)
        ctx.save_for_backward(x2, weight, rstd)
        ctx.shape = x.shape
        return y.view(x.shape)

    @staticmethod
    def backward(ctx, dy):
        x2, weight, rstd = ctx.saved_tensors
        dx, dw = _rmsnorm_backward(x2, weight, rstd, dy, None, ctx.shape)
        return dx, dw, None


def add_rms_norm(x: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor,
                 eps: float = 1e-6) -> Tuple[torch.Tensor, torch.Tensor]:
    """``r = x + delta`` (or ``x``) and ``rms_norm(r)``, one pass over the row.

    ``x`` is ``[rows, D]``; ``delta`` may cover only the first ``delta.shape[0]`` rows (the text rows of a
    full-attention layer in a hybrid stack, whose summary rows bypass the layer).
    """
    if not _cuda(x):
        if delta is not None and delta.shape[0] != x.shape[0]:
            pad = x.new_zeros((x.shape[0] - delta.shape[0],) + tuple(x.shape[1:]))
            delta = torch.cat([delta, pad], dim=0)
        return ref.add_rms_norm(x, delta, weight, eps)
    _require_bf16(x, delta, weight)
    x = x if x.is_contiguous() else x.contiguous()
    if delta is None:
        return x, _RmsNormFn.apply(x, weight, eps)
    delta = delta if delta.is_contiguous() else delta.contiguous()
    return _AddRmsNormFn.apply(x, delta, weight, eps)


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    if not _cuda(x):
        return ref.rms_norm(x, weight, eps)
    _require_bf16(x, weight)
    x = x if x.is_contiguous() else x.contiguous()
    return _RmsNormFn.apply(x, weight, eps)


# =============================================================================== QK-norm + RoPE
class _QkNormRopeFn(torch.autograd.Function):
    """Packed ``qkv`` rows ``[T, (Hq+2Hkv)*D]`` -> same layout with q, k normalised + rotated and v copied."""

    @staticmethod
    def forward(ctx, qkv, q_w, k_w, pos, Hq, Hkv, D, theta, eps, interleaved):
        T = qkv.shape[0]
        out = torch.empty((T, (Hq + 2 * Hkv) * D), dtype=qkv.dtype, device=qkv.device)
        rstd = torch.empty((T, Hq + Hkv), dtype=torch.float32, device=qkv.device)
        _lib.call("ksa_qknorm_rope_fwd", qkv, out, q_w, k_w, pos, rstd, qkv.stride(0), out.stride(0), T, Hq, Hkv, D,
                  float(theta), float(eps), int(interleaved), 1)
        ctx.save_for_backward(qkv, q_w, k_w, pos, rstd)
        ctx.cfg = (Hq, Hkv, D, theta, eps, interleaved)
        return out

    @staticmethod
    def backward(ctx, d_out):
        qkv, q_w, k_w, pos, rstd = ctx.saved_tensors
        Hq, Hkv, D, theta, eps, interleaved = ctx.cfg
        T = qkv.shape[0]
        d_out = d_out if d_out.is_contiguous() else d_out.contiguous()
        d_qkv = torch.empty_like(qkv)
        targets = []
        for w in (q_w, k_w):
            if w is None:
                targets.append(None)
                continue
            mg = getattr(w, "main_grad", None)
            if mg is not None:
                if not getattr(w, "_grad_written", False):
                    mg.zero_()
                    w._grad_written = True
                targets.append(mg)
            else:
                targets.append(torch.zeros(D, dtype=torch.float32, device=qkv.device))
        sinks = targets
        if _deterministic:     # the kernel's weight gradients are fp32 atomics: let them land in scratch vectors
            sinks = [None if t is None else torch.zeros(D, dtype=torch.float32, device=qkv.device) for t in targets]
        _lib.call("ksa_qknorm_rope_bwd", qkv, d_out, d_qkv, q_w, k_w, pos, rstd, sinks[0], sinks[1],
                  qkv.stride(0), d_out.stride(0), T, Hq, Hkv, D, float(theta), float(eps), int(interleaved), 1)
        if _deterministic:
            for t, g in zip(targets, _qk_norm_weight_grads(qkv, d_out, q_w, k_w, pos, *ctx.cfg)):
                if t is not None:
                    t.add_(g)
        grads = []
        for w, t in zip((q_w, k_w), targets):
            if w is None or getattr(w, "main_grad", None) is not None:
                grads.append(None)
            else:
                grads.append(t.to(w.dtype))
        return d_qkv, grads[0], grads[1], None, None, None, None, None, None, None


def _qk_norm_weight_grads(qkv, d_out, q_w, k_w, pos, Hq, Hkv, D, theta, eps, interleaved):
    """Gradients of the two QK-norm weight vectors in a fixed summation order (deterministic mode): the fp32 formulas
    differentiated by autograd, whose reductions over rows and heads use no atomics."""
    T = qkv.shape[0]
    with torch.enable_grad():
        q = qkv[:, :Hq * D].detach().float().reshape(1, T, Hq, D)
        k = qkv[:, Hq * D:(Hq + Hkv) * D].detach().float().reshape(1, T, Hkv, D)
        ws = [None if w is None else w.detach().float().requires_grad_(True) for w in (q_w, k_w)]
        qo, ko = ref.qk_norm_rope(q, k, ws[0], ws[1], pos, theta, eps, interleaved)
        dq = d_out[:, :Hq * D].float().reshape(1, T, Hq, D)
        dk = d_out[:, Hq * D:(Hq + Hkv) * D].float().reshape(1, T, Hkv, D)
        live = [w for w in ws if w is not None]
        got = list(torch.autograd.grad([qo, ko], live, [dq, dk], allow_unused=True)) if live else []
    out = []
    for w in ws:
        g = got.pop(0) if w is not None else None
        out.append(torch.zeros(D, dtype=torch.float32, device=qkv.device) if (w is not None and g is None) else g)
    return out


def qk_norm_rope_packed(qkv: torch.Tensor, q_w: Optional[torch.Tensor], k_w: Optional[torch.Tensor],
                        pos: torch.Tensor, Hq: int, Hkv: int, D: int, theta: float, eps: float = 1e-6,
                        interleaved: bool = False) -> torch.Tensor:
    """Per-head RMSNorm of q and k followed by RoPE, on packed projection rows.

    ``qkv`` is ``[T, (Hq+2Hkv)*D]`` (q heads | k heads | v heads), ``pos`` ``[T]``.  Returns the same
    layout: rotated q heads | rotated k heads | v heads unchanged, so that attention has one producer.
    """
    if not _cuda(qkv):
        T = qkv.shape[0]
        q = qkv[:, :Hq * D].reshape(1, T, Hq, D)
        k = qkv[:, Hq * D:(Hq + Hkv) * D].reshape(1, T, Hkv, D)
        q, k = ref.qk_norm_rope(q, k, q_w, k_w, pos, theta, eps, interleaved)
        return torch.cat([q.reshape(T, Hq * D), k.reshape(T, Hkv * D), qkv[:, (Hq + Hkv) * D:]], dim=1)
    _require_bf16(qkv, q_w, k_w)
    assert qkv.stride(1) == 1
    return _QkNormRopeFn.apply(qkv, q_w, k_w, pos.to(torch.int32), Hq, Hkv, D, theta, eps, interleaved)


def norm_linear(x: torch.Tensor, delta: Optional[torch.Tensor], norm_w: torch.Tensor, eps: float,
                weight: torch.Tensor, glu: bool = False):
    """``res = x + delta``; ``y = rms_norm(res, norm_w) @ weight.T`` (with ``glu``: ``swiglu`` of it, ``weight`` = gate
    rows then up rows).  Returns ``(res, y)``.  For at most 4 rows on a GPU without autograd (a decode step) this is
    one launch (``ksa_gemv_norm_bf16``: every CTA normalises the few activation rows itself while it stages them);
    everything else is ``add_rms_norm`` followed by the projection."""
    if (_cuda(x) and x.dim() == 2 and x.shape[0] <= 4 and x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16
            and not (torch.is_grad_enabled() and (x.requires_grad or weight.requires_grad))
            and x.stride(1) == 1 and weight.stride(1) == 1 and x.shape[1] % 8 == 0 and x.stride(0) % 8 == 0
            and weight.stride(0) % 8 == 0 and (delta is None or (delta.stride(1) == 1 and delta.stride(0) % 8 == 0
                                                                  and delta.dtype == torch.bfloat16))
            and (not glu or weight.shape[0] % 2 == 0)):
        M, K = x.shape
        N = weight.shape[0]
        res = torch.empty((M, K), dtype=torch.bfloat16, device=x.device) if delta is not None else x
        out = torch.empty((M, N // 2 if glu else N), dtype=torch.bfloat16, device=x.device)
        _lib.call("ksa_gemv_norm_bf16", x, delta, norm_w, res if delta is not None else None, weight, out, M, N, K,
                  x.stride(0), delta.stride(0) if delta is not None else K, res.stride(0), weight.stride(0),
                  out.stride(0), float(eps), delta.shape[0] if delta is not None else 0, int(glu))
        return res, out
    res, h = add_rms_norm(x, delta, norm_w, eps)
    return res, (linear_swiglu(h, weight) if glu else linear(h, weight))


def qk_norm_rope_decode(qkv: torch.Tensor, q_w: Optional[torch.Tensor], k_w: Optional[torch.Tensor],
                        pos: torch.Tensor, Hq: int, Hkv: int, D: int, theta: float, eps: float, interleaved: bool,
                        k_cache: torch.Tensor, v_cache: torch.Tensor, slots: torch.Tensor) -> torch.Tensor:
    """``qk_norm_rope_packed`` for the few rows of a decode step, with the cache append in the same kernel: the new K
    and V of row ``i < len(slots)`` (sequence ``i``) also go to ``k_cache`` / ``v_cache`` ``[B, Hkv, cap, D]`` at slot
    ``slots[i]`` (negative: not cached).  Inference only (no autograd)."""
    n = slots.numel()
    if _cuda(qkv) and D == 128 and qkv.dtype == torch.bfloat16 and qkv.stride(1) == 1:
        T = qkv.shape[0]
        out = torch.empty((T, (Hq + 2 * Hkv) * D), dtype=qkv.dtype, device=qkv.device)
        sl = slots.reshape(-1)
        sl = sl if sl.dtype == torch.int32 and sl.is_contiguous() else sl.to(torch.int32).contiguous()
        _lib.call("ksa_qknorm_rope_decode", qkv, out, q_w, k_w, pos.to(torch.int32), qkv.stride(0), out.stride(0), T, Hq,
                  Hkv, D, float(theta), float(eps), int(interleaved), k_cache, v_cache, sl, n, k_cache.shape[2])
        return out
    out = qk_norm_rope_packed(qkv, q_w, k_w, pos, Hq, Hkv, D, theta, eps, interleaved)
    k = out[:n, Hq * D:(Hq + Hkv) * D].reshape(n, Hkv, D)
    v = out[:n, (Hq + Hkv) * D:].reshape(n, Hkv, D)
    sl = slots.reshape(-1).tolist()
    for i, s_ in enumerate(sl):
        if s_ >= 0:
            k_cache[i, :, s_] = k[i]
            v_cache[i, :, s_] = v[i]
    return out


# =============================================================================== SwiGLU
class _SwiGluFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gu):
        F2 = gu.shape[-1]
        g2 = gu.reshape(-1, F2)
        out = torch.empty((g2.shape[0], F2 // 2), dtype=gu.dtype, device=gu.device)
        _lib.call("ksa_swiglu_fwd", g2, out, g2.shape[0], F2 // 2)
        ctx.save_for_backward(g2)
        ctx.shape = gu.shape
        return out.view(*gu.shape[:-1], F2 // 2)

    @staticmethod
    def backward(ctx, dout):
        (g2,) = ctx.saved_tensors
        d2 = dout.reshape(-1, dout.shape[-1])
        d2 = d2 if d2.is_contiguous() else d2.contiguous()
        dgu = torch.empty_like(g2)
        _lib.call("ksa_swiglu_bwd", g2, d2, dgu, g2.shape[0], g2.shape[1] // 2)
        return dgu.view(ctx.shape)


def swiglu(gate_up: torch.Tensor) -> torch.Tensor:
    """``silu(gate) * up`` with ``gate_up = [gate | up]`` along the last dimension."""
    if not _cuda(gate_up):
        return ref.swiglu(gate_up)
    _require_bf16(gate_up)
    gate_up = gate_up if gate_up.is_contiguous() else gate_up.contiguous()
    return _SwiGluFn.apply(gate_up)


def linear_swiglu(x: torch.Tensor, w13: torch.Tensor) -> torch.Tensor:
    """``swiglu(x @ w13.T)`` with ``w13 = [gate rows | up rows]``.  For at most 16 rows on a GPU without autograd (a
    decode step) the projection applies the activation itself (one kernel, ``ksa_gemv_swiglu_bf16``); everything else
    is the projection followed by ``swiglu``."""
    if (_cuda(x) and x.dim() == 2 and x.shape[0] <= 16 and x.dtype == torch.bfloat16 and w13.dtype == torch.bfloat16
            and not (torch.is_grad_enabled() and (x.requires_grad or w13.requires_grad))
            and x.stride(1) == 1 and w13.stride(1) == 1 and x.shape[1] % 8 == 0 and x.stride(0) % 8 == 0
            and w13.stride(0) % 8 == 0 and w13.shape[0] % 2 == 0):
        M, K = x.shape
        N = w13.shape[0]
        out = torch.empty((M, N // 2), dtype=torch.bfloat16, device=x.device)
        _lib.call("ksa_gemv_swiglu_bf16", x, w13, out, M, N, K, x.stride(0), w13.stride(0), out.stride(0))
        return out
    return swiglu(linear(x, w13))


# =============================================================================== embedding
class _EmbeddingFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, ids, table):
        flat = ids.reshape(-1).to(torch.int64).contiguous()
        D = table.shape[1]
        out = torch.empty((flat.numel(), D), dtype=table.dtype, device=table.device)
        _lib.call("ksa_embedding_fwd", flat, table, out, flat.numel(), D, table.shape[0])
        ctx.save_for_backward(flat, table)
        return out.view(*ids.shape, D)

    @staticmethod
    def backward(ctx, dout):
        flat, table = ctx.saved_tensors
        D = table.shape[1]
        d2 = dout.reshape(-1, D)
        d2 = d2 if d2.is_contiguous() else d2.contiguous()
        mg = getattr(table, "main_grad", None)
        if mg is not None:
            if not getattr(table, "_grad_written", False):
                mg.zero_()
                table._grad_written = True
            _embedding_grad(flat, d2, mg, D, table.shape[0])
            return None, None
        g = torch.zeros(table.shape, dtype=torch.float32, device=table.device)
        _embedding_grad(flat, d2, g, D, table.shape[0])
        return None, g.to(table.dtype)


def _embedding_grad(flat, d2, grad, D, vocab) -> None:
    """``grad[flat[i]] += d2[i]``.  The kernel adds rows with fp32 atomics; in deterministic mode the rows of every
    token id are brought together by a stable sort and summed one segment per thread, in row order, and the sums are
    added to distinct rows of ``grad``."""
    if not _deterministic:
        _lib.call("ksa_embedding_bwd", flat, d2, grad, flat.numel(), D, vocab)
        return
    order = torch.argsort(flat, stable=True)
    ids, counts = torch.unique_consecutive(flat[order], return_counts=True)
    sums = torch.segment_reduce(d2[order].float(), "sum", lengths=counts, axis=0, unsafe=True)
    grad[ids] += sums          # distinct rows: every element is written once


def embedding(ids: torch.Tensor, table: torch.Tensor) -> torch.Tensor:
    if not _cuda(table):
        return ref.embedding(ids, table)
    _require_bf16(table)
    return _EmbeddingFn.apply(ids, table)


# =============================================================================== attention
def _strides(t: torch.Tensor):
    """(row stride, batch stride) in elements of a ``[B, T, H, D]`` view with contiguous heads."""
    B, T, H, D = t.shape
    assert t.stride(3) == 1 and t.stride(2) == D, "heads must be contiguous blocks of head_dim"
    return t.stride(1), (t.stride(0) if B > 1 else t.stride(1) * max(T, 1))


_deterministic = os.environ.get("KSA_DETERMINISTIC", "0") == "1"


def set_deterministic(on: bool) -> None:
    """Bit-reproducible training step on one GPU.  Attention backward: two kernels that never accumulate across CTAs
    instead of the fused key-stationary one, whose dQ is summed with floating-point reductions in an order that
    varies between runs.  QK-norm weight gradients, the embedding gradient and the sum of squared gradients of the
    optimizer: summed in a fixed order instead of with fp32 atomics.  ``KSA_DETERMINISTIC=1`` sets the initial value.
    The reference kernel has the same switch (``flash_attn/cute/interface.py:801-811`` in the ``flash_attn_cute``
    wheel).  Not covered: the gradient-norm metric of the fused multi-GPU reduce + AdamW kernel (weights are)."""
    global _deterministic
    _deterministic = bool(on)


def is_deterministic() -> bool:
    return _deterministic


def _attn_bwd_text(q, k, v, ks, vs, o, do, lse, dq, dk, dv, dks, dvs, B, Hq, Hkv, D, Lq, Lk, Ns, *rest):
    """Text-query attention backward: the fused key-stationary kernel for head dim 128, else (and in deterministic
    mode) the two-kernel form.  ``rest`` = the 22 strides, the 7 layout integers, scale and the two fp32 partial
    buffers, in the order of the C entry points."""
    if B == 0 or Lq == 0:
        return
    if D == 128 and not _deterministic:
        lq_pad = (Lq + 127) // 128 * 128
        stats = torch.empty((2, B, Hq, lq_pad), dtype=torch.float32, device=q.device)
        dq32 = torch.empty((B, Lq, Hq, D), dtype=torch.float32, device=q.device)
        _lib.call("ksa_attn_bwd_fused", q, k, v, ks, vs, o, do, lse, stats, dq32, dq, dk, dv, dks, dvs,
                  B, Hq, Hkv, D, Lq, Lk, Ns, *rest)
    else:
        delta = torch.empty_like(lse)
        _lib.call("ksa_attn_bwd", q, k, v, ks, vs, o, do, lse, delta, dq, dk, dv, dks, dvs,
                  B, Hq, Hkv, D, Lq, Lk, Ns, *rest)



class _KsaAttentionFn(torch.autograd.Function):
    """Text + summary queries over text + summary keys (two-stream KSA); also plain causal attention."""

    @staticmethod
    def forward(ctx, q, k, v, qs, ks, vs, chunk, n_sum, window, tok_window, scale, q_off, k_off, s_off, seq_len,
                doc_start=None, doc_end=None):
        B, Lq, Hq, D = q.shape
        Lk, Hkv = k.shape[1], k.shape[2]
        has_sum = qs is not None and qs.shape[1] > 0
        Ns_k = ks.shape[1] if ks is not None else 0
        o = torch.empty((B, Lq, Hq, D), dtype=q.dtype, device=q.device)
        lse = torch.empty((B, Hq, Lq), dtype=torch.float32, device=q.device)
        qrs, qbs = _strides(q); krs, kbs = _strides(k); vrs, vbs = _strides(v)
        if Ns_k > 0:
            ksrs, ksbs = _strides(ks); vsrs, vsbs = _strides(vs)
        else:
            ksrs = ksbs = vsrs = vsbs = 0
        _lib.call("ksa_attn_fwd", q, k, v, ks if Ns_k > 0 else None, vs if Ns_k > 0 else None, o, lse,
                  B, Hq, Hkv, D, Lq, Lk, Ns_k, qrs, qbs, krs, kbs, vrs, vbs, ksrs, ksbs, vsrs, vsbs,
                  o.stride(1), o.stride(0), q_off, k_off, s_off, chunk, max(n_sum, 1), window, tok_window, float(scale),
                  doc_start, doc_end)
        os_ = lse_s = None
        if has_sum:
            Nq = qs.shape[1]
            os_ = torch.empty((B, Nq, Hq, D), dtype=q.dtype, device=q.device)
            lse_s = torch.empty((B, Hq, Nq), dtype=torch.float32, device=q.device)
            qsrs, qsbs = _strides(qs)
            chunk0 = q_off // chunk
            _lib.call("ksa_summary_attn_fwd", qs, k, v, ks, vs, os_, lse_s, B, Hq, Hkv, D, Nq, seq_len,
                      qsrs, qsbs, krs, kbs, vrs, vbs, ksrs, ksbs, vsrs, vsbs, os_.stride(1), os_.stride(0),
                      chunk, n_sum, chunk0, k_off, s_off, float(scale))
        ctx.save_for_backward(q, k, v, qs, ks, vs, o, lse, os_, lse_s)
        ctx.cfg = (chunk, n_sum, window, tok_window, scale, q_off, k_off, s_off, seq_len)
        ctx.docs = (doc_start, doc_end)
        if has_sum:
            return o, os_
        return o, None

    @staticmethod
    def backward(ctx, do, dos):
        q, k, v, qs, ks, vs, o, lse, os_, lse_s = ctx.saved_tensors
        chunk, n_sum, window, tok_window, scale, q_off, k_off, s_off, seq_len = ctx.cfg
        B, Lq, Hq, D = q.shape
        Lk, Hkv = k.shape[1], k.shape[2]
        Ns_k = ks.shape[1] if ks is not None else 0
        do = do if do.is_contiguous() else do.contiguous()
        dq = torch.empty_like(o)
        dk = torch.empty((B, Lk, Hkv, D), dtype=q.dtype, device=q.device)
        dv = torch.empty_like(dk)
        dks = dvs = None
        if Ns_k > 0:
            dks = torch.empty((B, Ns_k, Hkv, D), dtype=q.dtype, device=q.device)
            dvs = torch.empty_like(dks)
        part_k = part_v = None
        if Ns_k > 0 and os_ is not None and Lq > 0 and not _deterministic and _lib.attn_bwd_num_segments(Lq) > 1:
            part_k = torch.zeros((B, Ns_k, Hkv, D), dtype=torch.float32, device=q.device)
            part_v = torch.zeros_like(part_k)
        if Lq == 0:  # summary-only call: the text-query kernels do not run, start the key grads at zero
            dk.zero_(); dv.zero_()
            if dks is not None:
                dks.zero_(); dvs.zero_()
        qrs, qbs = _strides(q); krs, kbs = _strides(k); vrs, vbs = _strides(v)
        if Ns_k > 0:
            ksrs, ksbs = _strides(ks); vsrs, vsbs = _strides(vs)
            dksrs, dksbs = dks.stride(1), dks.stride(0)
        else:
            ksrs = ksbs = vsrs = vsbs = dksrs = dksbs = 0
        _attn_bwd_text(q, k, v, ks if Ns_k > 0 else None, vs if Ns_k > 0 else None, o, do, lse,
                       dq, dk, dv, dks, dvs, B, Hq, Hkv, D, Lq, Lk, Ns_k,
                       qrs, qbs, krs, kbs, vrs, vbs, ksrs, ksbs, vsrs, vsbs, o.stride(1), o.stride(0),
                       dq.stride(1), dq.stride(0), dk.stride(1), dk.stride(0), dv.stride(1), dv.stride(0),
                       dksrs, dksbs, dksrs, dksbs, q_off, k_off, s_off, chunk, max(n_sum, 1), window, tok_window,
                       float(scale), part_k, part_v, *ctx.docs)
        dqs = None
        if os_ is not None:
            Nq = qs.shape[1]
            dos = dos if dos.is_contiguous() else dos.contiguous()
            dqs = torch.empty_like(os_)
            qsrs, qsbs = _strides(qs)
            _lib.call("ksa_summary_attn_bwd", qs, k, v, ks, vs, os_, dos, lse_s, dqs, dk, dv, dks, dvs,
                      B, Hq, Hkv, D, Nq, seq_len, qsrs, qsbs, krs, kbs, vrs, vbs, ksrs, ksbs, vsrs, vsbs,
                      os_.stride(1), os_.stride(0), dqs.stride(1), dqs.stride(0), dk.stride(1), dk.stride(0),
                      dv.stride(1), dv.stride(0), dksrs, dksbs, dksrs, dksbs, chunk, n_sum, q_off // chunk,
                      k_off, s_off, float(scale), part_k, part_v, Ns_k)
        return (dq, dk, dv, dqs, dks, dvs) + (None,) * 11


def ksa_attention(q_t, k_t, v_t, q_s, k_s, v_s, chunk: int, n_sum: int, window: int,
                  scale: Optional[float] = None, skip_old_summary: bool = False,
                  q_off: int = 0, k_off: int = 0, s_off: int = 0, seq_len: Optional[int] = None):
    """Two-stream Kwai Summary Attention; returns ``(o_text, o_summary)``.

    ``q_off/k_off/s_off`` give the global index of local row 0 of the text queries, the text keys and
    the summary keys (context-parallel shards hold a halo of text keys and all older summary keys).
    ``seq_len`` is the global text length (defaults to ``k_off + Lk``).
    """
    D = q_t.shape[-1]
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    if not _cuda(q_t):
        assert q_off == 0 and k_off == 0 and s_off == 0, "the CPU path takes whole sequences"
        return ref.ksa_attention(q_t, k_t, v_t, q_s, k_s, v_s, chunk, n_sum, window, scale, skip_old_summary)
    _require_bf16(q_t, k_t, v_t, q_s, k_s, v_s)
    seq_len = seq_len if seq_len is not None else k_off + k_t.shape[1]
    if skip_old_summary:
        o_t, _ = _KsaAttentionFn.apply(q_t, k_t, v_t, None, None, None, chunk, n_sum, window, 0, scale,
                                       q_off, k_off, s_off, seq_len)
        _, o_s = _KsaAttentionFn.apply(q_t[:, :0], k_t, v_t, q_s, k_s, v_s, chunk, n_sum, window, 0, scale,
                                       q_off, k_off, s_off, seq_len)
        return o_t, o_s
    return _KsaAttentionFn.apply(q_t, k_t, v_t, q_s, k_s, v_s, chunk, n_sum, window, 0, scale,
                                 q_off, k_off, s_off, seq_len)


def causal_attention(q, k, v, scale: Optional[float] = None, window: int = -1,
                     cu_seqlens: Optional[torch.Tensor] = None, q_off: Optional[int] = None):
    """Causal attention (``window > 0``: keys with ``q - k < window``) on the same tensor-core kernel."""
    D = q.shape[-1]
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    if not _cuda(q):
        return ref.causal_attention(q, k, v, scale, window, cu_seqlens)
    _require_bf16(q, k, v)
    q_off = (k.shape[1] - q.shape[1]) if q_off is None else q_off
    doc_start = doc_end = None
    if cu_seqlens is not None:
        doc_start, doc_end = document_bounds(cu_seqlens, q.shape[0], q.shape[1], k.shape[1], q_off)
    o, _ = _KsaAttentionFn.apply(q, k, v, None, None, None, 128, 1, UNBOUNDED_WINDOW,
                                 window if window and window > 0 else 0, scale, q_off, 0, 0, k.shape[1],
                                 doc_start, doc_end)
    return o


def document_bounds(cu_seqlens: torch.Tensor, B: int, Lq: int, Lk: int, q_off: int = 0):
    """Per-row document bounds of a packed sequence for the attention kernels: ``cu_seqlens`` (``[n_docs + 1]``, token
    offsets as ``flash_attn_varlen_func`` takes them, the same packing for every sequence of the batch) ->
    ``(q_doc_start [B, Lq], k_doc_end [B, Lk])`` int32: the first token of each query's document and one past the
    last token of each key's document (``muse/layers/attention_utils.py:195-246`` passes the offsets themselves)."""
    cu = cu_seqlens.to(device="cuda" if torch.cuda.is_available() else cu_seqlens.device).to(torch.int64).reshape(-1)
    dev = cu.device
    tq = torch.arange(q_off, q_off + Lq, device=dev)
    tk = torch.arange(Lk, device=dev)
    dq = torch.bucketize(tq, cu[1:], right=True).clamp_(max=cu.numel() - 2)
    dk = torch.bucketize(tk, cu[1:], right=True).clamp_(max=cu.numel() - 2)
    start = cu[dq].to(torch.int32)[None, :].expand(B, -1).contiguous()
    end = cu[1:][dk].to(torch.int32)[None, :].expand(B, -1).contiguous()
    return start, end


def shard_causal_attention(q, k, v, scale: float, tok_window: int, q_off: int, k_off: int, seq_len: int):
    """Causal attention of a sequence shard: query row ``i`` is global position ``q_off + i``, key row ``j`` is
    ``k_off + j`` (context-parallel full-attention layers stage every earlier key in front of their own)."""
    _require_bf16(q, k, v)
    o, _ = _KsaAttentionFn.apply(q, k, v, None, None, None, 128, 1, UNBOUNDED_WINDOW,
                                 tok_window if tok_window and tok_window > 0 else 0, scale, q_off, k_off, 0, seq_len)
    return o


def _packed_views(qkv: torch.Tensor, B: int, T: int, Hq: int, Hkv: int, D: int, row0: int):
    rows = qkv[row0:row0 + B * T]
    q = rows[:, :Hq * D].view(B, T, Hq, D)
    k = rows[:, Hq * D:(Hq + Hkv) * D].view(B, T, Hkv, D)
    v = rows[:, (Hq + Hkv) * D:].view(B, T, Hkv, D)
    return q, k, v


class _PackedAttentionFn(torch.autograd.Function):
    """Attention on packed, rotated projection rows.

    ``qkv`` is ``[B*L + B*Ns, (Hq+2Hkv)*D]``: text rows of all sequences first, then summary rows.  The
    output is ``[B*L + B*Ns, Hq*D]`` in the same row order and the backward kernels write dq, dk, dv
    straight into the column blocks of one gradient buffer of the input's shape, so autograd never
    concatenates, pads or adds anything around the attention.  ``Ns = 0`` gives causal attention.
    """

    @staticmethod
    def forward(ctx, qkv, B, L, Ns, Hq, Hkv, D, chunk, n_sum, window, tok_window, scale, doc_start=None, doc_end=None):
        R = B * (L + Ns)
        assert qkv.shape[0] == R and qkv.stride(1) == 1
        q, k, v = _packed_views(qkv, B, L, Hq, Hkv, D, 0)
        out = torch.empty((R, Hq * D), dtype=qkv.dtype, device=qkv.device)
        o = out[:B * L].view(B, L, Hq, D)
        lse = torch.empty((B, Hq, L), dtype=torch.float32, device=qkv.device)
        rs = qkv.stride(0)
        if Ns > 0:
            qs, ks, vs = _packed_views(qkv, B, Ns, Hq, Hkv, D, B * L)
        else:
            qs = ks = vs = None
        _lib.call("ksa_attn_fwd", q, k, v, ks, vs, o, lse, B, Hq, Hkv, D, L, L, Ns,
                  rs, L * rs, rs, L * rs, rs, L * rs, rs, Ns * rs, rs, Ns * rs, Hq * D, L * Hq * D,
                  0, 0, 0, chunk, max(n_sum, 1), window, tok_window, float(scale), doc_start, doc_end)
        lse_s = None
        if Ns > 0:
            os_ = out[B * L:].view(B, Ns, Hq, D)
            lse_s = torch.empty((B, Hq, Ns), dtype=torch.float32, device=qkv.device)
            _lib.call("ksa_summary_attn_fwd", qs, k, v, ks, vs, os_, lse_s, B, Hq, Hkv, D, Ns, L,
                      rs, Ns * rs, rs, L * rs, rs, L * rs, rs, Ns * rs, rs, Ns * rs, Hq * D, Ns * Hq * D,
                      chunk, n_sum, 0, 0, 0, float(scale))
        ctx.save_for_backward(qkv, out, lse, lse_s)
        ctx.cfg = (B, L, Ns, Hq, Hkv, D, chunk, n_sum, window, tok_window, scale)
        ctx.docs = (doc_start, doc_end)
        return out

    @staticmethod
    def backward(ctx, dout):
        qkv, out, lse, lse_s = ctx.saved_tensors
        B, L, Ns, Hq, Hkv, D, chunk, n_sum, window, tok_window, scale = ctx.cfg
        dout = dout if dout.is_contiguous() else dout.contiguous()
        dqkv = torch.empty_like(qkv)
        rs, drs = qkv.stride(0), dqkv.stride(0)
        q, k, v = _packed_views(qkv, B, L, Hq, Hkv, D, 0)
        dq, dk, dv = _packed_views(dqkv, B, L, Hq, Hkv, D, 0)
        o = out[:B * L].view(B, L, Hq, D)
        do = dout[:B * L].view(B, L, Hq, D)
        part_k = part_v = None
        if Ns > 0:
            qs, ks, vs = _packed_views(qkv, B, Ns, Hq, Hkv, D, B * L)
            dqs, dks, dvs = _packed_views(dqkv, B, Ns, Hq, Hkv, D, B * L)
            if not _deterministic and _lib.attn_bwd_num_segments(L) > 1:
                part_k = torch.zeros((B, Ns, Hkv, D), dtype=torch.float32, device=qkv.device)
                part_v = torch.zeros_like(part_k)
        else:
            qs = ks = vs = dqs = dks = dvs = None
        _attn_bwd_text(q, k, v, ks, vs, o, do, lse, dq, dk, dv, dks, dvs,
                       B, Hq, Hkv, D, L, L, Ns,
                       rs, L * rs, rs, L * rs, rs, L * rs, rs, Ns * rs, rs, Ns * rs, Hq * D, L * Hq * D,
                       drs, L * drs, drs, L * drs, drs, L * drs, drs, Ns * drs, drs, Ns * drs,
                       0, 0, 0, chunk, max(n_sum, 1), window, tok_window, float(scale), part_k, part_v, *ctx.docs)
        if Ns > 0:
            os_ = out[B * L:].view(B, Ns, Hq, D)
            dos = dout[B * L:].view(B, Ns, Hq, D)
            _lib.call("ksa_summary_attn_bwd", qs, k, v, ks, vs, os_, dos, lse_s, dqs, dk, dv, dks, dvs,
                      B, Hq, Hkv, D, Ns, L, rs, Ns * rs, rs, L * rs, rs, L * rs, rs, Ns * rs, rs, Ns * rs,
                      Hq * D, Ns * Hq * D, drs, Ns * drs, drs, L * drs, drs, L * drs, drs, Ns * drs, drs, Ns * drs,
                      chunk, n_sum, 0, 0, 0, float(scale), part_k, part_v, Ns)
        return (dqkv,) + (None,) * 13


def attention_packed(qkv: torch.Tensor, B: int, L: int, Ns: int, Hq: int, Hkv: int, D: int, chunk: int = 128,
                     n_sum: int = 1, window: int = UNBOUNDED_WINDOW, tok_window: int = 0,
                     scale: Optional[float] = None, mode: str = "kernel",
                     cu_seqlens: Optional[torch.Tensor] = None) -> torch.Tensor:
    """KSA (``Ns > 0``) or causal (``Ns = 0``) attention on packed rotated rows; see :class:`_PackedAttentionFn`.

    ``mode`` selects the summary-attention implementation like the reference's ``summary_attention_mode``
    (``muse/layers/summary_attention_func.py:506-584``): ``"kernel"`` (the sm_100a kernels on a GPU, the dense oracle
    on CPU), ``"mask"`` (dense boolean mask, plain PyTorch, any device) or ``"block"`` (query blocks with gathered
    keys, plain PyTorch, any device).  ``cu_seqlens`` (causal attention only): documents packed into the sequence; a
    query sees keys of its own document only."""
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    if mode not in ("kernel", "mask", "block"):
        raise ValueError(f"unknown summary attention mode {mode!r}")
    if not _cuda(qkv) or (Ns > 0 and mode != "kernel"):
        q, k, v = _packed_views(qkv, B, L, Hq, Hkv, D, 0)
        if Ns > 0:
            qs, ks, vs = _packed_views(qkv, B, Ns, Hq, Hkv, D, B * L)
            fn = ref.ksa_attention_blockwise if mode == "block" else ref.ksa_attention
            o_t, o_s = fn(q, k, v, qs, ks, vs, chunk, n_sum, window, scale)
            return torch.cat([o_t.reshape(B * L, Hq * D), o_s.reshape(B * Ns, Hq * D)], dim=0)
        return ref.causal_attention(q, k, v, scale, tok_window if tok_window > 0 else -1,
                                    cu_seqlens).reshape(B * L, Hq * D)
    _require_bf16(qkv)
    docs = (None, None)
    if cu_seqlens is not None:
        if Ns > 0:
            raise ValueError("packed documents apply to causal attention only: summary tokens are inserted without "
                             "regard to document boundaries")
        docs = document_bounds(cu_seqlens, B, L, L)
    return _PackedAttentionFn.apply(qkv, B, L, Ns, Hq, Hkv, D, chunk, n_sum, window, tok_window, scale, *docs)


# =============================================================================== fused linear + cross entropy
class _LinearCrossEntropyFn(torch.autograd.Function):
    """lm_head GEMM + softmax CE, chunked over tokens so that only one chunk of logits exists."""

    @staticmethod
    def forward(ctx, hidden, weight, labels, ignore_index, chunk_tokens):
        T, D = hidden.shape
        V = weight.shape[0]
        dev = hidden.device
        labels = labels.reshape(-1).to(torch.int64).contiguous()
        stats = torch.empty(2, dtype=torch.float32, device=dev)
        _lib.call("ksa_count_valid", labels, T, ignore_index, 1.0, stats)
        inv_n = stats[1:2]
        row_loss = torch.empty(T, dtype=torch.float32, device=dev)
        need_h = ctx.needs_input_grad[0]
        need_w = ctx.needs_input_grad[1]
        dh = torch.empty_like(hidden) if need_h else None
        mg = getattr(weight, "main_grad", None)
        if need_w:
            if mg is not None:
                dw, acc0 = mg, getattr(weight, "_grad_written", False)
            else:
                dw, acc0 = torch.empty((V, D), dtype=torch.float32, device=dev), False
        logits = torch.empty((min(chunk_tokens, T), V), dtype=torch.bfloat16, device=dev)
        for i, s in enumerate(range(0, T, chunk_tokens)):
            e = min(T, s + chunk_tokens)
            lg = logits[: e - s]
            gemm(hidden[s:e], weight, out=lg)
            _lib.call("ksa_cross_entropy", lg, labels[s:e], row_loss[s:e], inv_n, e - s, V, lg.stride(0),
                      ignore_index, int(need_h or need_w))
            if need_h:
                gemm(lg, weight, b_mn_major=True, out=dh[s:e])
            if need_w:
                gemm(lg, hidden[s:e], a_mn_major=True, b_mn_major=True, out=dw, accumulate=(acc0 or i > 0))
        if need_w and mg is not None:
            weight._grad_written = True
        loss = (row_loss.sum() * inv_n).reshape(())
        ctx.dh = dh
        ctx.dw = None if (not need_w or mg is not None) else dw
        ctx.w_dtype = weight.dtype
        return loss

    @staticmethod
    def backward(ctx, dloss):
        # Gradients were produced for d(loss) = 1 in forward; scale by the incoming gradient.
        dh = ctx.dh * dloss.to(ctx.dh.dtype) if ctx.dh is not None else None
        dw = (ctx.dw * dloss).to(ctx.w_dtype) if ctx.dw is not None else None
        return dh, dw, None, None, None


def linear_cross_entropy(hidden: torch.Tensor, weight: torch.Tensor, labels: torch.Tensor,
                         ignore_index: int = -100, chunk_tokens: int = 2048) -> torch.Tensor:
    """Mean next-token CE of ``hidden @ weight.T``; logits never exist for more than one token chunk.

    On CUDA the gradients w.r.t. ``hidden`` and ``weight`` are computed during the forward pass (the
    softmax is turned into the gradient in place), assuming the loss is the root of the backward pass
    up to a scalar factor; with ``main_grad`` on the weight that factor must be 1.
    """
    if not _cuda(hidden):
        return ref.linear_cross_entropy(hidden, weight, labels, ignore_index)
    _require_bf16(hidden, weight)
    h2 = hidden.reshape(-1, hidden.shape[-1])
    h2 = h2 if h2.is_contiguous() else h2.contiguous()
    return _LinearCrossEntropyFn.apply(h2, weight, labels, ignore_index, chunk_tokens)


# =============================================================================== optimiser
def adamw_step(master, grad, m, v, out_bf16, hyper, beta1, beta2, eps, weight_decay, clip_value=0.0,
               sumsq: Optional[torch.Tensor] = None) -> None:
    """Fused AdamW over a flat fp32 buffer; ``hyper`` = device tensor ``[lr, 1-b1^t, 1-b2^t, grad_scale]``."""
    if not _cuda(master):
        lr, bc1, bc2, gs = [float(x) for x in hyper.tolist()]
        g = grad.float() * gs
        if clip_value > 0:
            g = g.clamp(-clip_value, clip_value)
        if sumsq is not None:
            sumsq += (g * g).sum()
        m.mul_(beta1).add_(g, alpha=1 - beta1)
        v.mul_(beta2).addcmul_(g, g, value=1 - beta2)
        master.mul_(1 - lr * weight_decay)
        master.addcdiv_(m / bc1, (v / bc2).sqrt_().add_(eps), value=-lr)
        if out_bf16 is not None:
            out_bf16.copy_(master)
        return
    n = master.numel()
    if _deterministic and sumsq is not None:     # the kernel adds its blocks' sums with an atomic: sum in a fixed order
        g = grad * hyper[3]
        if clip_value > 0:
            g = g.clamp_(-clip_value, clip_value)
        sumsq += (g * g).sum()
        sumsq = None
    _lib.call("ksa_adamw", master, grad, m, v, out_bf16, n, hyper, float(beta1), float(beta2), float(eps),
              float(weight_decay), float(clip_value), sumsq)


__all__ = [
    "gemm", "linear", "dual_linear", "attention_packed", "rms_norm", "add_rms_norm", "qk_norm_rope_packed", "qk_norm_rope_decode", "swiglu", "linear_swiglu", "norm_linear", "embedding",
    "ksa_attention", "causal_attention", "linear_cross_entropy", "adamw_step", "UNBOUNDED_WINDOW",
    "SummaryLayout", "get_layout",
]
