"""ctypes binding of the in-tree sm_100a kernel library (``ksa_b200/_lib/libksa_b200.so``).

The library exports plain C entry points that take raw device pointers, sizes,
strides in elements and a CUDA stream.  ``call(name, *args)`` launches one on
torch's current stream and raises with the library's own message on error.  On
a machine with a GPU a missing library is an error, never a silent fallback.
"""
from __future__ import annotations

import ctypes
import os
import threading
from pathlib import Path
from typing import Dict, Optional, Sequence

import torch

_LIB_PATH = Path(__file__).resolve().parent.parent / "_lib" / "libksa_b200.so"
_lib: Optional[ctypes.CDLL] = None

P, I, L, F = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float

# name -> argument ctypes (the trailing stream pointer included)
_SIGNATURES: Dict[str, Sequence] = {
    "ksa_gemm_bf16": [P, P, P, I, I, I, L, L, L, I, I, I, I, F, I, P],
    "ksa_gemm2_bf16": [P, P, P, I, I, I, L, L, L, I, I, I, I, F, P],
    "ksa_gemm2_gather_bf16": [P, P, P, I, I, I, L, L, L, I, I, F, P, I, I, L, P, P, ctypes.c_uint, P, I, L, P],
    "ksa_gemm2_scatter_bf16": [P, P, I, I, I, L, L, L, P, I, I, P],
    "ksa_gemv_bf16": [P, P, P, I, I, I, L, L, L, P],
    "ksa_gemv_swiglu_bf16": [P, P, P, I, I, I, L, L, L, P],
    "ksa_gemv_norm_bf16": [P, P, P, P, P, P, I, I, I, L, L, L, L, L, F, I, I, P],
    "ksa_rmsnorm_fwd": [P, P, P, P, P, P, I, I, F, I, P],
    "ksa_rmsnorm_bwd": [P, P, P, P, P, P, P, P, I, I, I, P],
    "ksa_qknorm_rope_fwd": [P, P, P, P, P, P, L, L, I, I, I, I, F, F, I, I, P],
    "ksa_qknorm_rope_decode": [P, P, P, P, P, L, L, I, I, I, I, F, F, I, P, P, P, I, I, P],
    "ksa_qknorm_rope_bwd": [P, P, P, P, P, P, P, P, P, L, L, I, I, I, I, F, F, I, I, P],
    "ksa_swiglu_fwd": [P, P, L, I, P],
    "ksa_swiglu_bwd": [P, P, P, L, I, P],
    "ksa_embedding_fwd": [P, P, P, L, I, L, P],
    "ksa_embedding_bwd": [P, P, P, L, I, L, P],
    "ksa_count_valid": [P, L, I, F, P, P],
    "ksa_cross_entropy": [P, P, P, P, L, I, L, I, I, P],
    "ksa_adamw": [P, P, P, P, P, L, P, F, F, F, F, F, P, P],
    "ksa_cast_f32_bf16": [P, P, L, P],
    "ksa_attn_fwd": [P] * 7 + [I] * 7 + [L] * 12 + [I] * 7 + [F, P, P, P],
    "ksa_attn_bwd": [P] * 14 + [I] * 7 + [L] * 22 + [I] * 7 + [F, P, P, P, P, P],
    "ksa_attn_bwd_fused": [P] * 15 + [I] * 7 + [L] * 22 + [I] * 7 + [F, P, P, P, P, P],
    "ksa_attn_fwd_cp": [P, P, P, I, I, I, I, I, L, L, L, L, P, I, I, P, I, I, L, L, L, P, P, ctypes.c_uint, I, I, I, I, I, I, F, P],
    "ksa_attn_bwd_fused_cp": [P] * 11 + [I] * 5 + [L] * 14 + [P, I, I, P, I, I, L, L, L, P, P, ctypes.c_uint, P, P, L, L, L,
                                                              I, I, I, I, I, I, F, P, P, P],
    "ksa_cp_fold_return": [P, P, I, I, I, L, L, L, L, P, I, ctypes.c_uint, P],
    "ksa_summary_attn_fwd": [P] * 7 + [I] * 6 + [L] * 12 + [I] * 5 + [F, P],
    "ksa_summary_attn_bwd": [P] * 13 + [I] * 6 + [L] * 22 + [I] * 5 + [F, P, P, I, P],
    "ksa_decode_attn": [P] * 8 + [I] * 8 + [F, P, P],
    "ksa_kv_cache_append": [P] * 5 + [I] * 5 + [L, L, P],
    "ksa_kv_cache_move": [P] * 5 + [I] * 5 + [P],
    "ksa_peer_gather": [P, I, I, L, I, P, P, ctypes.c_uint, I, P],
    "ksa_peer_reduce_adamw": [P, I, I, L, L, P, P, P, P, P, F, F, F, F, F, P, P, P, ctypes.c_uint, I, P],
    "ksa_signal_set": [P, I, P, ctypes.c_uint, P],
    "ksa_signal_wait": [P, I, P, ctypes.c_uint, P],
    "ksa_peer_copy": [P, P, L, P, P, ctypes.c_uint, I, P],
    "ksa_peer_add_bf16": [P, P, L, P, P, ctypes.c_uint, I, P],
    "ksa_peer_copy2d": [P, L, P, L, L, L, P, P, ctypes.c_uint, I, P],
    "ksa_tp_allreduce_add_rmsnorm": [P, P, P, P, I, I, P, P, P, I, I, I, F, P, P, P],
    "ksa_tp_reduce_scatter_add_rmsnorm": [P, P, P, P, I, I, P, P, P, I, I, I, F, P, P, I, I, P, P],
    "ksa_symm_alloc": [P, L],
    "ksa_symm_free": [P],
    "ksa_ipc_get_handle": [P, P],
    "ksa_ipc_open_handle": [P, P],
    "ksa_ipc_close": [P],
}


def lib_path() -> Path:
    return _LIB_PATH


def available() -> bool:
    return _LIB_PATH.exists()


def load() -> ctypes.CDLL:
    global _lib
    if _lib is not None:
        return _lib
    if not _LIB_PATH.exists():
        raise RuntimeError(
            f"{_LIB_PATH} is missing: build it with `python -m ksa_b200.csrc.build` (needs nvcc); "
            "CUDA tensors cannot be processed without the sm_100a kernel library")
    lib = ctypes.CDLL(str(_LIB_PATH), mode=ctypes.RTLD_LOCAL)
    lib.ksa_last_error.restype = ctypes.c_char_p
    lib.ksa_read_status.argtypes = [I]
    lib.ksa_read_status.restype = I
    lib.ksa_rmsnorm_bwd_parts.argtypes = [I]
    lib.ksa_rmsnorm_bwd_parts.restype = I
    lib.ksa_attn_bwd_num_segments.argtypes = [I]
    lib.ksa_attn_bwd_num_segments.restype = I
    lib.ksa_set_dependent_launch.argtypes = [I]
    lib.ksa_set_dependent_launch.restype = I
    for name, sig in _SIGNATURES.items():
        fn = getattr(lib, name, None)
        if fn is not None:
            fn.argtypes = list(sig)
            fn.restype = I
    _lib = lib
    return lib


_STATUS_TEXT = {
    1: "a consumer timed out waiting for a TMA-filled stage",
    2: "the TMA producer timed out waiting for a free stage",
    3: "an epilogue/softmax warp timed out waiting for an MMA commit",
    4: "the MMA issuer timed out waiting for the epilogue to drain TMEM",
    5: "timed out waiting for a flag written by another CTA or GPU",
    6: "the MMA issuer timed out waiting for the softmax warps",
    7: "a kernel rejected its arguments",
}


def _ptr(x):
    if x is None:
        return None
    if isinstance(x, torch.Tensor):
        if not x.is_cuda:  # a host pointer handed to a kernel is an illegal access on the device
            raise TypeError("a CPU tensor was passed to an sm_100a kernel entry point")
        return x.data_ptr()
    return x


# kernels launched by one call of an entry point (default 1)
_KERNELS_PER_CALL = {"ksa_attn_bwd": 2, "ksa_attn_bwd_fused": 3, "ksa_attn_bwd_fused_cp": 3, "ksa_rmsnorm_bwd": 2}
_launch_count = 0


def call(name: str, *args) -> None:
    """Launch entry point ``name`` on the current CUDA stream (appended as the last argument)."""
    global _launch_count
    lib = load()
    fn = getattr(lib, name)
    stream = torch.cuda.current_stream().cuda_stream
    rc = fn(*[_ptr(a) for a in args], stream)
    if rc != 0:
        raise RuntimeError(f"{name} failed ({rc}): {lib.ksa_last_error().decode()}")
    _launch_count += _KERNELS_PER_CALL.get(name, 1)


def call_nostream(name: str, *args) -> None:
    """Call an entry point that takes no stream argument (set-up routines)."""
    lib = load()
    rc = getattr(lib, name)(*[_ptr(a) for a in args])
    if rc != 0:
        raise RuntimeError(f"{name} failed ({rc}): {lib.ksa_last_error().decode()}")


_tls = threading.local()


def attach_pair_gather(job: dict) -> None:
    """Hand a parameter all-gather to the next CTA-pair GEMM of this thread that can carry it (``ops.gemm`` runs it
    inside that launch with ``ksa_gemm2_gather_bf16``).  The caller must call ``flush_pair_gather`` before the gathered
    data is needed, in case no such GEMM came by.

    ``job``: ``peers`` (ctypes pointer array), ``world``, ``rank``, ``shard_bytes``, ``ready`` (address of the ready
    flags), ``epoch`` (device tensor or None), ``epoch_add``, ``done`` (int32 device tensor of ``GATHER_COUNTERS``
    completion counters), ``base`` / ``nbytes`` (this rank's copy of the gathered buffer), ``min_flops`` (smallest
    GEMM that may carry it)."""
    flush_pair_gather()
    _tls.pair_gather = job


def pair_gather_pending() -> bool:
    return getattr(_tls, "pair_gather", None) is not None


def peek_pair_gather() -> Optional[dict]:
    return getattr(_tls, "pair_gather", None)


def take_pair_gather() -> Optional[dict]:
    job, _tls.pair_gather = getattr(_tls, "pair_gather", None), None
    return job


def flush_pair_gather() -> None:
    """Run a gather that is still waiting for a GEMM as a kernel of its own, now."""
    job = take_pair_gather()
    if job is not None:
        call("ksa_peer_gather", job["peers"], job["world"], job["rank"], job["shard_bytes"], 1, job["ready"],
             job["epoch"], job["epoch_add"], 32)


def launch_count() -> int:
    """Kernels of this library launched (or captured into a graph) so far in this process."""
    return _launch_count


def count_launches(fn) -> int:
    """Run ``fn()`` and return how many kernels of this library it launched."""
    before = _launch_count
    fn()
    return _launch_count - before


def call_on(name: str, stream: int, *args) -> None:
    lib = load()
    rc = getattr(lib, name)(*[_ptr(a) for a in args], stream)
    if rc != 0:
        raise RuntimeError(f"{name} failed ({rc}): {lib.ksa_last_error().decode()}")


def check_status(clear: bool = True) -> None:
    """Synchronise and raise if any kernel's bounded wait gave up since the last check."""
    st = load().ksa_read_status(1 if clear else 0)
    if st != 0:
        if st & 0xFF == 8:
            raise RuntimeError(f"kernel status {st}: a debug-build bounds check failed at source line {st >> 8}")
        raise RuntimeError(f"kernel status {st}: {_STATUS_TEXT.get(st, 'unknown')}")


def set_peer_wait_ms(ms: int) -> None:
    """Limit of device-side waits on flags written by other GPUs (current device; default 10 s, or KSA_PEER_WAIT_MS)."""
    if load().ksa_set_peer_wait_ms(int(ms)) != 0:
        raise RuntimeError("could not set the peer wait limit")


def set_dependent_launch(on: bool) -> bool:
    """Switch dependent launches of the decode-step kernels (programmatic stream serialization: a kernel may start
    while its predecessor on the stream still runs and waits for it on the device) on or off; returns the previous
    setting.  The inference engine switches it on around a decode step; training leaves it off."""
    return load().ksa_set_dependent_launch(1 if on else 0) != 0


GATHER_COUNTERS = 32   # int32 completion counters a ``ksa_gemm2_gather_bf16`` launch uses (8 shards x 4 segments)


def attn_bwd_num_segments(lq: int) -> int:
    return load().ksa_attn_bwd_num_segments(lq)


def rmsnorm_bwd_parts(rows: int) -> int:
    return load().ksa_rmsnorm_bwd_parts(rows)
