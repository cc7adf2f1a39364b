"""Symmetric memory over NVLink: one device allocation per rank, mapped into every peer.

Each rank allocates a buffer with the kernel library (``cudaMalloc``), exports a CUDA IPC handle, and opens the
handles of the other ranks (exchanged once over the process group), so that kernels can issue loads and stores to
any rank's copy through ordinary pointers.  ``SymmetricBuffer.tensor`` is a torch view of the local copy;
``peer_ptrs`` lists the device pointers of all copies (own copy included) in rank order, and ``ptr_array`` is the
same as a ctypes array for the C entry points.  Signal pads are small symmetric ``uint32`` buffers used as
cross-GPU flags (release-store by the producer, bounded acquire-wait by the consumer).

The reference has no such layer (it calls NCCL through FSDP2 for everything); this is the substrate for the fused
compute+communication kernels.
"""
from __future__ import annotations

import ctypes
from typing import List, Optional

import torch
import torch.distributed as dist

from ..ops import _lib


class _CudaArray:
    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3}


class SymmetricBuffer:
    def __init__(self, nbytes: int, group: Optional[dist.ProcessGroup] = None, device: Optional[torch.device] = None):
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.nbytes = int((nbytes + 255) // 256 * 256)
        self.device = device or torch.device("cuda", torch.cuda.current_device())
        _lib.load()
        out = ctypes.c_void_p()
        _lib.call_nostream("ksa_symm_alloc", ctypes.byref(out), self.nbytes)
        self.local_ptr = out.value
        self._opened: List[int] = []
        self.peer_ptrs: List[int] = [0] * self.world
        self.peer_ptrs[self.rank] = self.local_ptr
        if self.world > 1:
            handle = (ctypes.c_ubyte * 64)()
            _lib.call_nostream("ksa_ipc_get_handle", self.local_ptr, ctypes.cast(handle, ctypes.c_void_p))
            handles: List[Optional[bytes]] = [None] * self.world
            dist.all_gather_object(handles, bytes(handle), group=group)
            for r, h in enumerate(handles):
                if r == self.rank:
                    continue
                buf = (ctypes.c_ubyte * 64).from_buffer_copy(h)
                p = ctypes.c_void_p()
                _lib.call_nostream("ksa_ipc_open_handle", ctypes.cast(buf, ctypes.c_void_p), ctypes.byref(p))
                self.peer_ptrs[r] = p.value
                self._opened.append(p.value)
            dist.barrier(group=group)
        self.ptr_array = (ctypes.c_void_p * self.world)(*self.peer_ptrs)
        self._bytes = torch.as_tensor(_CudaArray(self.local_ptr, self.nbytes), device=self.device)

    def view(self, dtype: torch.dtype, offset_bytes: int = 0, numel: Optional[int] = None) -> torch.Tensor:
        """Typed view of the local copy starting ``offset_bytes`` in."""
        item = torch.empty((), dtype=dtype).element_size()
        numel = (self.nbytes - offset_bytes) // item if numel is None else numel
        return self._bytes[offset_bytes:offset_bytes + numel * item].view(dtype)

    def offset_ptr_array(self, offset_bytes: int):
        """ctypes array of every rank's pointer advanced by ``offset_bytes``."""
        return (ctypes.c_void_p * self.world)(*[p + offset_bytes for p in self.peer_ptrs])

    def close(self) -> None:
        if self.local_ptr is None:
            return
        torch.cuda.synchronize(self.device)
        if self.world > 1 and dist.is_initialized():
            dist.barrier(group=self.group)
        for p in self._opened:
            _lib.call_nostream("ksa_ipc_close", p)
        self._opened = []
        self._bytes = None
        _lib.call_nostream("ksa_symm_free", self.local_ptr)
        self.local_ptr = None


class SignalPad:
    """``n`` uint32 flags per rank in symmetric memory; ``flag_ptrs(i)`` addresses flag ``i`` on every rank."""

    def __init__(self, n: int, group=None, device=None):
        self.buf = SymmetricBuffer(n * 4, group, device)
        self.n = n
        self.flags = self.buf.view(torch.int32, 0, n)
        self.world, self.rank = self.buf.world, self.buf.rank

    def flag_ptrs(self, index: int):
        return self.buf.offset_ptr_array(index * 4)

    def local_ptr(self, index: int) -> int:
        return self.buf.local_ptr + index * 4

    def set_on_all(self, index: int, epoch: Optional[torch.Tensor], add: int = 0) -> None:
        """After all prior work of the current stream, store ``epoch[0] + add`` to flag ``index`` on every rank.

        ``epoch`` is a device ``int32``/``uint32`` scalar tensor (or ``None`` for 0): reading the value on the device
        keeps a captured CUDA graph valid while the step counter advances."""
        _lib.call("ksa_signal_set", self.flag_ptrs(index), self.world, epoch, add)

    def wait_local(self, index: int, n: int, epoch: Optional[torch.Tensor], add: int = 0) -> None:
        _lib.call("ksa_signal_wait", self.local_ptr(index), n, epoch, add)

    def close(self) -> None:
        self.flags = None
        self.buf.close()
