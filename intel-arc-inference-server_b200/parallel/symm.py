"""Symmetric device buffers and the wire objects the fused collective kernels take.

Every rank allocates the same buffer, the ranks exchange CUDA IPC handles over the process
group, and each rank maps all peers' buffers: kernels then store into a peer's landing buffer
with ordinary global stores that cross NVLink.  The reference does the same for its two cards
with Level Zero IPC allocations and a landing buffer per direction
(src/runtime/tp_engine.h:26-96, src/runtime/tp_protocol.h:1-157).

``SymmBuffer``   one allocation per rank + the peers' mapped addresses.
``Wire``         landing buffer + flag array + call counters for one family of collectives, and
                 the device table of all ranks' addresses that kernels read.
"""
from __future__ import annotations

import ctypes
from typing import List, Optional, Sequence

import torch

from ..ops import lib as K

MAX_RANKS = 8


class _DevMem:
    """``__cuda_array_interface__`` view of raw device memory so torch can wrap it without a copy."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 2}


class SymmBuffer:
    def __init__(self, nbytes: int, group=None, device: Optional[torch.device] = None):
        import torch.distributed as dist
        self.nbytes = (int(nbytes) + 255) // 256 * 256
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.device = device or torch.device("cuda", torch.cuda.current_device())
        L = K.lib()
        p = ctypes.c_void_p()
        with torch.cuda.device(self.device):
            K._check(L.b2_symm_alloc(ctypes.byref(p), ctypes.c_ulonglong(self.nbytes)), "symm_alloc")
            self.local_ptr = p.value
            self.ptrs: List[int] = [0] * self.world
            self.ptrs[self.rank] = self.local_ptr
            self._opened: List[int] = []
            if self.world > 1:
                hb = L.b2_ipc_handle_bytes()
                h = (ctypes.c_ubyte * hb)()
                K._check(L.b2_ipc_get(ctypes.c_void_p(self.local_ptr), h), "ipc_get")
                mine = torch.tensor(list(bytes(h)), dtype=torch.uint8, device=self.device)
                allh = [torch.empty_like(mine) for _ in range(self.world)]
                dist.all_gather(allh, mine, group=group)
                for r in range(self.world):
                    if r == self.rank:
                        continue
                    hr = (ctypes.c_ubyte * hb)(*allh[r].cpu().tolist())
                    q = ctypes.c_void_p()
                    K._check(L.b2_ipc_open(hr, ctypes.byref(q)), f"ipc_open(rank {r})")
                    self.ptrs[r] = q.value
                    self._opened.append(q.value)
                dist.barrier(group=group)
        self._bytes = torch.as_tensor(_DevMem(self.local_ptr, self.nbytes), device=self.device)

    def view(self, dtype: torch.dtype, offset: int = 0, numel: Optional[int] = None) -> torch.Tensor:
        """Tensor over this rank's own part."""
        es = torch.empty((), dtype=dtype).element_size()
        n = (self.nbytes - offset) // es if numel is None else numel
        return self._bytes[offset: offset + n * es].view(dtype)

    def close(self):
        L = K.lib()
        torch.cuda.synchronize(self.device)
        self._bytes = None
        for q in self._opened:
            L.b2_ipc_close(ctypes.c_void_p(q))
        self._opened = []
        if self.local_ptr:
            L.b2_symm_free(ctypes.c_void_p(self.local_ptr))
            self.local_ptr = 0


class Wire:
    """One landing buffer, flag array and epoch counters; ``table`` is what the kernels are given."""

    def __init__(self, land_bytes: int, n_flags: int, n_epochs: int, group=None, device=None):
        self.flag_off = (land_bytes + 4095) // 4096 * 4096
        self.buf = SymmBuffer(self.flag_off + n_flags * 4 + 4096, group, device)
        self.world, self.rank, self.device = self.buf.world, self.buf.rank, self.buf.device
        tab = [0] * (2 * MAX_RANKS)
        for r in range(self.world):
            tab[r] = self.buf.ptrs[r]
            tab[MAX_RANKS + r] = self.buf.ptrs[r] + self.flag_off
        self.table = torch.tensor(tab, dtype=torch.int64, device=self.device)
        self.epoch = torch.zeros(max(n_epochs, 1), dtype=torch.int32, device=self.device)
        self.land = self.buf.view(torch.float32, 0, land_bytes // 4)
        self.flags = self.buf.view(torch.int32, self.flag_off, n_flags)

    def close(self):
        self.land = self.flags = None
        self.buf.close()


class TpWires:
    """The wires of a tensor-parallel decode step: the row-parallel fold (o and down projections share
    one, calls alternate), the vocabulary-parallel arg-max and a general small all-reduce."""

    def __init__(self, hidden: int, mcap: int, group=None, device=None):
        import torch.distributed as dist
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.mcap, self.hidden, self.group = mcap, hidden, group
        nb = (hidden + 127) // 128
        w = self.world
        self.fold = Wire(2 * w * mcap * hidden * 4, 2 * w * nb, nb, group, device)
        self.head = Wire(2 * w * mcap * 2 * 4, 2 * w * mcap, mcap, group, device)
        nblk = (hidden + 1023) // 1024
        self.sum = Wire(2 * w * mcap * hidden * 4, 2 * w * mcap * nblk, mcap * nblk, group, device)

    def reset(self):
        """Flags and call counters back to zero (after a failure; every rank must do it before the next step)."""
        for x in (self.fold, self.head, self.sum):
            x.flags.zero_()
            x.epoch.zero_()

    def close(self):
        for x in (self.fold, self.head, self.sum):
            x.close()
