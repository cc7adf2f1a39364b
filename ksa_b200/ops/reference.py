"""Plain PyTorch implementations of every op: the CPU path and the numerics oracle.

Each function is differentiable through ordinary autograd and computes in
fp32 internally, returning the input dtype.  GPU tests compare the sm_100a
kernels against these run in fp32.
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch
import torch.nn.functional as F

from .layout import two_stream_masks


# ---------------------------------------------------------------- norms
def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    """``x * rsqrt(mean(x^2) + eps) * weight`` in fp32 (``muse/layers/rms_norm.py:67-80``)."""
    xf = x.float()
    y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    return (y * weight.float()).to(x.dtype)


def add_rms_norm(x: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor,
                 eps: float = 1e-6) -> Tuple[torch.Tensor, torch.Tensor]:
    """Residual add fused with the following norm: returns ``(x + delta, norm(x + delta))``."""
    r = x if delta is None else (x.float() + delta.float()).to(x.dtype)
    return r, rms_norm(r, weight, eps)


# ---------------------------------------------------------------- RoPE
def rope_cos_sin(pos: torch.Tensor, head_dim: int, theta: float) -> Tuple[torch.Tensor, torch.Tensor]:
    """fp32 cos/sin tables ``[..., head_dim/2]`` for integer positions ``pos``."""
    half = head_dim // 2
    inv = 1.0 / (theta ** (torch.arange(0, half, device=pos.device, dtype=torch.float32) * 2.0 / head_dim))
    ang = pos.to(torch.float32)[..., None] * inv
    return ang.cos(), ang.sin()


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """Half-split (HF) rotary: ``x*cos + rotate_half(x)*sin``; ``x`` is ``[..., T, H, D]``.

    ``cos``/``sin`` are ``[..., T, D/2]`` and broadcast over heads
    (``muse/layers/position_embeddings.py:245-293``).
    """
    xf = x.float()
    half = x.shape[-1] // 2
    x1, x2 = xf[..., :half], xf[..., half:]
    c, s = cos[..., None, :], sin[..., None, :]
    return torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], dim=-1).to(x.dtype)


def apply_rope_interleaved(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """Llama-style rotary on adjacent pairs (``muse/layers/position_embeddings.py:48-162``)."""
    xf = x.float().reshape(*x.shape[:-1], -1, 2)
    c, s = cos[..., None, :], sin[..., None, :]
    out = torch.stack([xf[..., 0] * c - xf[..., 1] * s, xf[..., 1] * c + xf[..., 0] * s], dim=-1)
    return out.flatten(-2).to(x.dtype)


def qk_norm_rope(q: torch.Tensor, k: torch.Tensor, q_weight: Optional[torch.Tensor],
                 k_weight: Optional[torch.Tensor], pos: torch.Tensor, theta: float,
                 eps: float = 1e-6, interleaved: bool = False) -> Tuple[torch.Tensor, torch.Tensor]:
    """Per-head RMSNorm on q and k, *then* RoPE (``muse/models/qwen3/_layers.py:267-301``).

    ``q``: ``[B, T, Hq, D]``, ``k``: ``[B, T, Hkv, D]``, ``pos``: ``[T]`` or ``[B, T]``.
    """
    if q_weight is not None:
        q = rms_norm(q, q_weight, eps)
    if k_weight is not None:
        k = rms_norm(k, k_weight, eps)
    cos, sin = rope_cos_sin(pos, q.shape[-1], theta)
    rot = apply_rope_interleaved if interleaved else apply_rope
    return rot(q, cos, sin), rot(k, cos, sin)


# ---------------------------------------------------------------- MLP
def swiglu(gate_up: torch.Tensor) -> torch.Tensor:
    """``silu(gate) * up`` for ``gate_up = [gate | up]`` along the last dim."""
    g, u = gate_up.float().chunk(2, dim=-1)
    return (F.silu(g) * u).to(gate_up.dtype)


def linear(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    return F.linear(x, weight, bias)


# ---------------------------------------------------------------- attention
def _expand_kv(k: torch.Tensor, n_rep: int) -> torch.Tensor:
    return k if n_rep == 1 else k.repeat_interleave(n_rep, dim=2)


def _masked_attention(q, k, v, mask, scale):
    """q ``[B,Tq,H,D]``, k/v ``[B,Tk,H,D]``, mask ``[Tq,Tk]`` bool. fp32. Returns (out, lse)."""
    s = torch.einsum("bqhd,bkhd->bhqk", q.float(), k.float()) * scale
    s = s.masked_fill(~mask, float("-inf"))
    lse = torch.logsumexp(s, dim=-1)
    p = torch.exp(s - lse[..., None])
    p = torch.nan_to_num(p, nan=0.0)
    o = torch.einsum("bhqk,bkhd->bqhd", p, v.float())
    return o, lse


def ksa_attention(q_t, k_t, v_t, q_s, k_s, v_s, chunk: int, n_sum: int, window: int,
                  scale: Optional[float] = None, skip_old_summary: bool = False):
    """Two-stream Kwai Summary Attention, dense-mask fp32 reference.

    Text streams ``[B, L, H, D]``; summary streams ``[B, ceil(L/C)*S, H, D]``.
    Returns ``(o_t, o_s)`` in the input dtype.  Semantics: a text query sees its
    own chunk causally, the previous ``window`` chunks' text, and the summaries
    of every older chunk; a summary query sees its own chunk's text and the
    summaries of that chunk up to itself (``summary_attn/mask.py:19-31`` in the reference's ``summary_attn`` wheel).
    ``skip_old_summary`` drops the old-summary keys (pure sliding-chunk attention).
    """
    B, L, Hq, D = q_t.shape
    n_rep = Hq // k_t.shape[2]
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    tt, ts, st, ss = two_stream_masks(L, chunk, n_sum, window, device=q_t.device, n_summary_rows=q_s.shape[1])
    if skip_old_summary:
        ts = torch.zeros_like(ts)
    k_all = torch.cat([_expand_kv(k_t, n_rep), _expand_kv(k_s, n_rep)], dim=1)
    v_all = torch.cat([_expand_kv(v_t, n_rep), _expand_kv(v_s, n_rep)], dim=1)
    o_t, _ = _masked_attention(q_t, k_all, v_all, torch.cat([tt, ts], dim=1), scale)
    o_s, _ = _masked_attention(q_s, k_all, v_all, torch.cat([st, ss], dim=1), scale)
    return o_t.to(q_t.dtype), o_s.to(q_s.dtype)


def ksa_attention_blockwise(q_t, k_t, v_t, q_s, k_s, v_s, chunk: int, n_sum: int, window: int,
                            scale: Optional[float] = None, q_block: int = 4096):
    """The same attention as :func:`ksa_attention` without the ``O(L^2)`` mask: the queries are processed in blocks of
    ``q_block`` rows, and every block gathers only the keys it can see (the text of its own chunks and of the
    ``window`` chunks before them, the summaries of older chunks) with a compact mask of that size (the reference's
    ``"block"`` mode, ``muse/layers/summary_attention_func.py:194-457``).  Memory is ``O(q_block * (window * chunk +
    q_block + L / chunk * n_sum))``; plain PyTorch, differentiable, any device."""
    B, L, Hq, D = q_t.shape
    Ns = q_s.shape[1]
    n_rep = Hq // k_t.shape[2]
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    q_block = max(chunk, q_block // chunk * chunk)                 # whole chunks per block
    dev = q_t.device
    out_t = []
    for q0 in range(0, L, q_block):
        q1 = min(L, q0 + q_block)
        c0, c1 = q0 // chunk, (q1 - 1) // chunk                    # first and last chunk of the block
        k0 = max(0, c0 - window) * chunk                           # first visible text key
        s1 = min(max(0, c1 - window) * n_sum, Ns)                  # summaries of chunks older than the last chunk's window
        tq = torch.arange(q0, q1, device=dev)[:, None]
        tk = torch.arange(k0, q1, device=dev)[None, :]
        m_text = (tk <= tq) & (tq // chunk - tk // chunk <= window)
        sk = torch.arange(s1, device=dev)[None, :] // max(n_sum, 1)
        m_sum = (tq // chunk - sk) > window
        k_all = torch.cat([_expand_kv(k_t[:, k0:q1], n_rep), _expand_kv(k_s[:, :s1], n_rep)], dim=1)
        v_all = torch.cat([_expand_kv(v_t[:, k0:q1], n_rep), _expand_kv(v_s[:, :s1], n_rep)], dim=1)
        o, _ = _masked_attention(q_t[:, q0:q1], k_all, v_all, torch.cat([m_text, m_sum], dim=1), scale)
        out_t.append(o)
    out_s = []
    s_block = max(n_sum, q_block // chunk * n_sum)                 # summary rows of q_block text rows
    for r0 in range(0, Ns, s_block):
        r1 = min(Ns, r0 + s_block)
        c0, c1 = r0 // n_sum, (r1 - 1) // n_sum
        t0, t1 = c0 * chunk, min(L, (c1 + 1) * chunk)              # the text of the block's own chunks
        sq = torch.arange(r0, r1, device=dev)[:, None]
        tk = torch.arange(t0, t1, device=dev)[None, :]
        sk = torch.arange(r0, r1, device=dev)[None, :]
        m_text = (sq // n_sum) == (tk // chunk)
        m_sum = ((sq // n_sum) == (sk // n_sum)) & ((sk % n_sum) <= (sq % n_sum))
        k_all = torch.cat([_expand_kv(k_t[:, t0:t1], n_rep), _expand_kv(k_s[:, r0:r1], n_rep)], dim=1)
        v_all = torch.cat([_expand_kv(v_t[:, t0:t1], n_rep), _expand_kv(v_s[:, r0:r1], n_rep)], dim=1)
        o, _ = _masked_attention(q_s[:, r0:r1], k_all, v_all, torch.cat([m_text, m_sum], dim=1), scale)
        out_s.append(o)
    o_t = torch.cat(out_t, dim=1).to(q_t.dtype)
    o_s = (torch.cat(out_s, dim=1) if out_s else q_s.new_zeros(q_s.shape)).to(q_s.dtype)
    return o_t, o_s


def causal_attention(q, k, v, scale: Optional[float] = None, window: int = -1,
                     cu_seqlens: Optional[torch.Tensor] = None):
    """Causal (optionally token-sliding-window, optionally packed-document) attention.

    ``window > 0`` keeps keys with ``q - k < window`` (FA2 ``window_size=(w-1, 0)``
    convention of ``muse/layers/attention_utils.py:222-246``).
    """
    B, Tq, Hq, D = q.shape
    Tk = k.shape[1]
    n_rep = Hq // k.shape[2]
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    qi = torch.arange(Tk - Tq, Tk, device=q.device)[:, None]
    ki = torch.arange(Tk, device=q.device)[None, :]
    mask = ki <= qi
    if window is not None and window > 0:
        mask = mask & (qi - ki < window)
    if cu_seqlens is not None:
        doc = torch.bucketize(torch.arange(Tk, device=q.device), cu_seqlens[1:].to(q.device), right=True)
        mask = mask & (doc[Tk - Tq:, None] == doc[None, :])
    o, _ = _masked_attention(q, _expand_kv(k, n_rep), _expand_kv(v, n_rep), mask, scale)
    return o.to(q.dtype)


def interleaved_ksa_attention(q, k, v, chunk: int, n_sum: int, window: int, scale=None):
    """The reference's own formulation: one interleaved sequence + dense mask + softmax.

    Used only to prove that the two-stream form above computes the same function.
    """
    from .layout import dense_interleaved_mask
    B, T, Hq, D = q.shape
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    mask = dense_interleaved_mask(T, chunk, n_sum, window, device=q.device)
    n_rep = Hq // k.shape[2]
    o, _ = _masked_attention(q, _expand_kv(k, n_rep), _expand_kv(v, n_rep), mask, scale)
    return o.to(q.dtype)


def decode_attention(q, k_cache, v_cache, lengths: torch.Tensor, start: Optional[torch.Tensor] = None,
                     scale: Optional[float] = None):
    """One-or-few-token decode over a contiguous cache slice per sequence.

    ``q`` ``[B, Tq, Hq, D]``; caches ``[B, Hkv, cap, D]``; sequence ``b`` attends
    slots ``[start[b], start[b]+lengths[b])`` with no mask inside the slice
    (``examples/pretrain/hf_template/modeling_qwen3sa.py:402-434``).
    """
    B, Tq, Hq, D = q.shape
    Hkv, cap = k_cache.shape[1], k_cache.shape[2]
    n_rep = Hq // Hkv
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    start = torch.zeros_like(lengths) if start is None else start
    slot = torch.arange(cap, device=q.device)[None, :]
    valid = (slot >= start[:, None]) & (slot < (start + lengths)[:, None])       # [B, cap]
    kf = k_cache.float().repeat_interleave(n_rep, dim=1)
    vf = v_cache.float().repeat_interleave(n_rep, dim=1)
    s = torch.einsum("bqhd,bhkd->bhqk", q.float(), kf) * scale
    s = s.masked_fill(~valid[:, None, None, :], float("-inf"))
    p = torch.softmax(s, dim=-1)
    return torch.einsum("bhqk,bhkd->bqhd", p, vf).to(q.dtype)


# ---------------------------------------------------------------- losses
def cross_entropy(logits: torch.Tensor, labels: torch.Tensor, ignore_index: int = -100):
    """fp32 token cross entropy: returns ``(sum_loss, n_valid)`` (``muse/losses/ce.py:32-140``)."""
    loss = F.cross_entropy(logits.float().reshape(-1, logits.shape[-1]), labels.reshape(-1),
                           ignore_index=ignore_index, reduction="sum")
    return loss, (labels != ignore_index).sum()


def linear_cross_entropy(hidden: torch.Tensor, weight: torch.Tensor, labels: torch.Tensor,
                         ignore_index: int = -100) -> torch.Tensor:
    """Mean CE of ``hidden @ weight.T`` against ``labels`` over non-ignored tokens."""
    logits = F.linear(hidden, weight)
    s, n = cross_entropy(logits, labels, ignore_index)
    return s / n.clamp(min=1)


def embedding(ids: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    return F.embedding(ids, weight)


# ---------------------------------------------------------------- optimiser
def adamw_step_(master: torch.Tensor, grad: torch.Tensor, m: torch.Tensor, v: torch.Tensor,
                lr: float, beta1: float, beta2: float, eps: float, weight_decay: float, step: int,
                grad_scale: float = 1.0, clip_value: float = 0.0,
                out_bf16: Optional[torch.Tensor] = None) -> torch.Tensor:
    """In-place decoupled AdamW on fp32 state; returns the sum of squared (scaled, clipped) gradients.

    ``clip_value > 0`` clamps each gradient element to ``[-clip, clip]`` first
    (the reference clips by value, ``muse/training/common.py:122-141``).
    """
    g = grad.float() * grad_scale
    if clip_value > 0:
        g = g.clamp(-clip_value, clip_value)
    sq = (g * g).sum()   # of the clipped gradients: the reference clips before it measures the norm
    m.mul_(beta1).add_(g, alpha=1 - beta1)
    v.mul_(beta2).addcmul_(g, g, value=1 - beta2)
    bc1 = 1 - beta1 ** step
    bc2 = 1 - beta2 ** step
    master.mul_(1 - lr * weight_decay)
    denom = (v / bc2).sqrt_().add_(eps)
    master.addcdiv_(m / bc1, denom, value=-lr)
    if out_bf16 is not None:
        out_bf16.copy_(master)
    return sq
