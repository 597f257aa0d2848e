"""Pinned host buffers for small arrays that go to the device every step."""
from __future__ import annotations

import torch


class PinnedRing:
    """Pinned int32 host buffers used in turn, so that a copy to the device never makes the host wait
    for the device's earlier work (a copy from pageable memory does).  A buffer is reused only after the
    copy that read it has completed: ``take`` gives (turn, buffer), and ``copied(turn)`` is called once
    the copy has been put on the stream."""

    def __init__(self, device, count: int = 4):
        self.device = torch.device(device)
        self.pinned = self.device.type == "cuda"
        self.buffers = [None] * count
        self.events = [None] * count
        self.turn = 0

    def take(self, n_ints: int):
        i = self.turn
        self.turn = (self.turn + 1) % len(self.buffers)
        if self.events[i] is not None:
            self.events[i].synchronize()
        buf = self.buffers[i]
        if buf is None or buf.numel() < n_ints:
            size = max(1024, 1 << (n_ints - 1).bit_length())
            buf = torch.empty(size, dtype=torch.int32, pin_memory=self.pinned)
            self.buffers[i] = buf
        return i, buf[:n_ints]

    def copied(self, i: int) -> None:
        if self.pinned:
            event = torch.cuda.Event()
            event.record()
            self.events[i] = event
