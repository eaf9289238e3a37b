"""Pinned host staging buffers for non-blocking host-to-device copies.

``tensor.copy_(pinned, non_blocking=True)`` only QUEUES the copy: it runs when the stream gets to it, which can be
long after the call returns (behind a CUDA graph or a prompt chunk that is still computing).  Until then the pinned
buffer must not change, or the device receives the later contents.  ``Staged`` keeps a small ring of pinned buffers
with one CUDA event each: ``begin()`` hands out the next buffer after waiting for the copy that last read it,
``push()`` queues the copy and records the event.  With a ring of two the host stays one step ahead of the device
instead of waiting for it.
"""
from __future__ import annotations

from typing import List, Optional

import torch


class Staged:
    def __init__(self, shape, dtype, depth: int = 2):
        pin = torch.cuda.is_available()
        self._hosts: List[torch.Tensor] = []
        for _ in range(max(1, depth)):
            t = torch.zeros(shape, dtype=dtype)
            self._hosts.append(t.pin_memory() if pin else t)
        self._events: List[Optional[torch.cuda.Event]] = [None] * len(self._hosts)
        self._i = 0

    @property
    def host(self) -> torch.Tensor:
        """The buffer handed out by the last ``begin()``."""
        return self._hosts[self._i]

    def begin(self) -> torch.Tensor:
        """The next host buffer, safe to overwrite: the copy that last read it has run."""
        self._i = (self._i + 1) % len(self._hosts)
        ev = self._events[self._i]
        if ev is not None:
            ev.synchronize()
        return self._hosts[self._i]

    def push(self, dst: torch.Tensor, src: Optional[torch.Tensor] = None):
        """Queue ``dst.copy_(src)`` (``src``: a view of the current host buffer; default the whole buffer)."""
        dst.copy_(self.host if src is None else src, non_blocking=True)
        if dst.is_cuda:
            ev = self._events[self._i]
            if ev is None:
                ev = self._events[self._i] = torch.cuda.Event()
            ev.record(torch.cuda.current_stream(dst.device))
