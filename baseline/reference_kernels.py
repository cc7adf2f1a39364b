"""The reference's own sm_100 attention kernels (its ``flash_attn_cute`` and ``summary_attn`` wheels), for same-box
comparisons in ``kernel_bench attn --compare-ref``.  One GPU only: the copy under ``baseline/_ref_kernels`` does not
travel to multi-GPU calls, and every tensor these kernels see lives on this GPU.

* dense causal attention: ``flash_attn.cute.interface.flash_attn_func`` (forward; forward + backward);
* Kwai Summary Attention: the wheel's ``SummaryAttnFunc`` builds its block-sparsity lists with tile sizes chosen for
  Hopper (128 x 64 forward), which the sm_100 kernels refuse ("must be a multiple of 256"); :func:`summary_attention`
  calls the same two wheel functions (``SummaryAttnFunc._get_cached_value`` and ``_flash_attn_fwd`` /
  ``_flash_attn_bwd``) with 256 x 128 lists and 128 x 128 kernel tiles instead.  No wheel file is edited.

Every entry point returns ``(callable, None)`` or ``(None, "<why it cannot run>")``; the wheels pin
``nvidia-cutlass-dsl < 4.4`` and ``quack-kernels == 0.2.4`` while this image has 4.5.0 and 0.4.1, so the import or the
JIT compilation may fail, and that text is what gets reported.
"""
from __future__ import annotations

import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
KERNELS = os.path.join(HERE, "_ref_kernels")


def _short(e: BaseException) -> str:
    return " ".join(f"{type(e).__name__}: {e}".split())[:300]


def _import():
    if not os.path.isdir(os.path.join(KERNELS, "flash_attn", "cute")):
        raise RuntimeError(f"{KERNELS} is not installed on this machine (1-GPU calls only)")
    if KERNELS not in sys.path:
        sys.path.insert(0, KERNELS)
    import flash_attn
    cute_dir = os.path.join(KERNELS, "flash_attn")
    if cute_dir not in list(flash_attn.__path__):
        flash_attn.__path__.append(cute_dir)
    import flash_attn.cute.interface as iface
    return iface


def dense_causal():
    """``fn(q, k, v) -> o`` (``[B, L, H, D]`` bf16, differentiable) on the reference's sm_100 kernels."""
    try:
        iface = _import()
    except BaseException as e:  # noqa: BLE001
        return None, _short(e)

    def fn(q, k, v):
        out = iface.flash_attn_func(q, k, v, causal=True)
        return out[0] if isinstance(out, tuple) else out
    return fn, None


def summary_attention(chunk: int, n_sum: int, window: int):
    """``fn(q, k, v, summary_pos) -> o`` on the interleaved layout of the reference (``[1, L + L/C*S, H, D]``), GQA
    expanded by the caller as the reference's layer does; sm_100 tile sizes as described above."""
    try:
        iface = _import()
        import torch
        from summary_attn.interface import SummaryAttnFunc
    except BaseException as e:  # noqa: BLE001
        return None, _short(e)

    class _Sm100SummaryAttn(torch.autograd.Function):
        @staticmethod
        def forward(ctx, q, k, v):
            sparse, mask_mod = SummaryAttnFunc._get_cached_value(q.shape[1], k.shape[1], chunk, n_sum, window,
                                                                 is_fwd=True, m_block_size=256, n_block_size=128)
            out, lse = iface._flash_attn_fwd(q, k, v, mask_mod=mask_mod, block_sparse_tensors=sparse, m_block_size=128,
                                             n_block_size=128)
            ctx.save_for_backward(q, k, v, out, lse)
            return out

        @staticmethod
        def backward(ctx, dout):
            q, k, v, out, lse = ctx.saved_tensors
            sparse, mask_mod = SummaryAttnFunc._get_cached_value(q.shape[1], k.shape[1], chunk, n_sum, window,
                                                                 is_fwd=False, m_block_size=256, n_block_size=128)
            return iface._flash_attn_bwd(q, k, v, out, dout, lse, mask_mod=mask_mod, block_sparse_tensors=sparse,
                                         m_block_size=128, n_block_size=128)

    def fn(q, k, v, summary_pos):
        import torch
        k = torch.cat((k[:, summary_pos, :], k), dim=1)      # the wrapper's summary-prefix copy (interface.py:276-278)
        v = torch.cat((v[:, summary_pos, :], v), dim=1)
        return _Sm100SummaryAttn.apply(q, k, v)
    return fn, None
