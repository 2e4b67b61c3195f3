"""Device-memory log at named points (reference optimus/memory_profiler.py:5-41)."""
from __future__ import annotations

import torch

GB = 1024 ** 3


class MemoryLogInfo:
    def __init__(self, tag, init=False):
        self.tag = tag
        if init or not torch.cuda.is_available():
            self.allocated = self.reserved = self.max_allocated = 0.0
        else:
            self.allocated = torch.cuda.memory_allocated() / GB
            self.reserved = torch.cuda.memory_reserved() / GB
            self.max_allocated = torch.cuda.max_memory_allocated() / GB


class MemoryTracker:
    """Prints allocated / reserved / peak memory and the delta to the previous entry, on the
    ranks with dp = ep = pp = 0 only."""

    def __init__(self, pmap=None):
        self.pmap = pmap
        self.entries = [MemoryLogInfo("init", init=True)]

    def _enabled(self):
        p = self.pmap
        return p is None or (p.dp_ind == 0 and getattr(p, "ep_ind", 0) == 0 and getattr(p, "pp_ind", 0) == 0)

    def log(self, tag):
        if not self._enabled():
            return
        cur = MemoryLogInfo(tag)
        self.print_current_entry(cur, self.entries[-1])
        self.entries.append(cur)

    def print_current_entry(self, cur, prev):
        print(f"[Memory] {cur.tag:40s} allocated {cur.allocated:8.3f} GB ({cur.allocated - prev.allocated:+8.3f}), "
              f"reserved {cur.reserved:8.3f} GB ({cur.reserved - prev.reserved:+8.3f}), "
              f"peak {cur.max_allocated:8.3f} GB", flush=True)

    def print_all_entries(self):
        for prev, cur in zip(self.entries[:-1], self.entries[1:]):
            self.print_current_entry(cur, prev)
