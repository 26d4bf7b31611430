"""Small integer arrays from the host to the device in one copy.

A step describes its batch with a handful of short int32 arrays (slots, row
offsets, token ids, page-table rows).  Pinning a new host buffer for each of
them, or copying each from pageable memory, costs the host more than
everything else it does for a step of a few thousand tokens, and the device
waits for it.  Here the arrays are laid side by side in one of a few pinned
buffers that are kept and used in turn, and leave in one asynchronous copy; a
buffer is written again only after the copy that last left from it has ended.
The copy holds the values as they were when ``upload`` was called, whatever
the host does to its own tables afterwards.
"""

from __future__ import annotations

from typing import List, Sequence

import torch


class HostStaging:
    def __init__(self, device, depth: int = 4):
        self.device = torch.device(device)
        self._buffers: List = [None] * depth
        self._events: List = [None] * depth   # the event after the copy that last left from each buffer
        self._turn = 0

    def upload(self, parts: Sequence[torch.Tensor]) -> List[torch.Tensor]:
        """The parts (int32 tensors on the host, any shape) on the device, as views of one tensor, in their order."""
        flat = [p.reshape(-1) for p in parts]
        if self.device.type != "cuda":
            whole = torch.cat(flat) if flat else torch.empty(0, dtype=torch.int32)
        else:
            n = sum(int(p.numel()) for p in flat)
            i = self._turn
            self._turn = (i + 1) % len(self._buffers)
            if self._events[i] is not None:
                self._events[i].synchronize()
            buf = self._buffers[i]
            if buf is None or buf.numel() < n:
                buf = self._buffers[i] = torch.empty(max(2 * n, 4096), dtype=torch.int32, pin_memory=True)
            if n:
                torch.cat(flat, out=buf[:n])
            whole = buf[:n].to(self.device, non_blocking=True)
            self._events[i] = torch.cuda.Event()
            self._events[i].record()
        out, at = [], 0
        for p in parts:
            out.append(whole[at:at + p.numel()].view(p.shape))
            at += p.numel()
        return out
