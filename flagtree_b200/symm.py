"""Peer-mapped ("symmetric") device buffers for the GEMM + reduce-scatter workspace.

Every rank allocates a buffer of the same size and obtains a device pointer to every peer's
buffer.  Two providers, tried in order:
  1. torch.distributed._symmetric_memory (cuMem allocation + handle exchange done by torch);
  2. CUDA IPC through the C ABI (ftb_ipc_alloc / ftb_ipc_open), handles exchanged with
     all_gather_object.
The exchange itself only needs a process group, so it is testable on CPU with a fake provider.
"""
from __future__ import annotations

import ctypes as C
from typing import Callable, List, Optional, Sequence

import torch
import torch.distributed as dist


def exchange_handles(local_handle: bytes, group=None) -> List[bytes]:
    """all_gather of one opaque handle per rank (rank order)."""
    world = dist.get_world_size(group)
    out: List[Optional[bytes]] = [None] * world
    dist.all_gather_object(out, local_handle, group=group)
    return [bytes(h) for h in out]


class SymmetricBuffer:
    """`nbytes` of zeroed device memory on every rank; `ptrs[i]` = this process's pointer to rank i's."""

    def __init__(self, nbytes: int, group=None, device: Optional[torch.device] = None, provider: str = "auto",
                 _alloc: Optional[Callable] = None, _open: Optional[Callable] = None):
        self.group = group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        self.nbytes = int(nbytes)
        self.ptrs: List[int] = []
        self.mc_ptr: int = 0            # NVSwitch multicast address of all ranks' buffers (0 = none)
        self._keep = None
        self._opened: List[int] = []
        self._owned: Optional[int] = None
        self.provider = None
        errors = []
        if _alloc is not None:                       # injected provider (CPU tests)
            self._init_handles(_alloc, _open)
            self.provider = "injected"
            return
        if provider in ("auto", "symm_mem"):
            try:
                self._init_symm_mem(device)
                self.provider = "symm_mem"
            except Exception as e:                   # noqa: BLE001 - fall through to IPC
                errors.append(f"symm_mem: {e!r}")
                if provider == "symm_mem":
                    raise
        if self.provider is None:
            try:
                self._init_ipc()
                self.provider = "cuda_ipc"
            except Exception as e:                   # noqa: BLE001
                errors.append(f"cuda_ipc: {e!r}")
                raise RuntimeError("no symmetric-memory provider worked: " + "; ".join(errors))
        dist.barrier(group)

    # -- providers
    def _init_symm_mem(self, device):
        import torch.distributed._symmetric_memory as symm_mem
        t = symm_mem.empty(self.nbytes, dtype=torch.uint8, device=device)
        t.zero_()
        torch.cuda.synchronize()
        g = self.group if self.group is not None else dist.group.WORLD
        hdl = symm_mem.rendezvous(t, g)
        ptrs = list(hdl.buffer_ptrs)
        assert len(ptrs) == self.world and ptrs[self.rank] == t.data_ptr()
        self.ptrs = [int(p) for p in ptrs]
        try:
            self.mc_ptr = int(getattr(hdl, "multicast_ptr", 0) or 0)
        except Exception:               # noqa: BLE001 - multicast is optional
            self.mc_ptr = 0
        self._keep = (t, hdl)

    def _init_ipc(self):
        from . import _lib
        lib = _lib.load()

        def alloc(nbytes):
            ptr = C.c_void_p()
            handle = (C.c_uint8 * 64)()
            _lib.check(lib.ftb_ipc_alloc(C.c_int64(nbytes), C.byref(ptr), handle), "ftb_ipc_alloc")
            return int(ptr.value), bytes(handle)

        def open_(handle):
            ptr = C.c_void_p()
            buf = (C.c_uint8 * 64).from_buffer_copy(handle)
            _lib.check(lib.ftb_ipc_open(buf, C.byref(ptr)), "ftb_ipc_open")
            return int(ptr.value)

        self._init_handles(alloc, open_)

    def _init_handles(self, alloc, open_):
        local_ptr, handle = alloc(self.nbytes)
        self._owned = local_ptr
        handles = exchange_handles(handle, self.group)
        for r, h in enumerate(handles):
            if r == self.rank:
                self.ptrs.append(local_ptr)
            else:
                p = open_(h)
                self._opened.append(p)
                self.ptrs.append(p)

    @property
    def local_ptr(self) -> int:
        return self.ptrs[self.rank]

    def close_peers(self):
        """Drops this process's mappings of the peers' buffers (the owners still hold the memory).  Callers put a
        group barrier before this (no kernel of any rank touches the buffers any more) and another one between
        this and `close` (no peer still maps the memory that is about to be freed)."""
        if self.provider == "cuda_ipc":
            from . import _lib
            lib = _lib.load()
            for p in self._opened:
                lib.ftb_ipc_close(C.c_void_p(p))
        self._opened = []

    def close(self):
        """Releases this rank's own buffer (and, if `close_peers` was not called, the peers' mappings first)."""
        self.close_peers()
        if self.provider == "cuda_ipc" and self._owned is not None:
            from . import _lib
            _lib.load().ftb_ipc_free(C.c_void_p(self._owned))
        self._owned, self._keep = None, None
