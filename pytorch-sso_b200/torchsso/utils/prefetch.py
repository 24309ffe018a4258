"""Double-buffered host -> device input pipeline for a closure that reads fixed device tensors.

A closure replayed from a CUDA graph (``GraphedClosure``) reads its batch from fixed tensors, so
every step starts by copying a batch into them.  Done on the compute stream, the copy from pinned
host memory (19 MB for 32 ImageNet-sized images) sits in front of the step; here it runs on a copy
stream into one of two staging buffers while the previous step computes, and the step itself starts
with a device-to-device copy.  Every batch still crosses the bus exactly once.
"""
from __future__ import annotations

from typing import Iterable, Sequence

import torch


class BatchPrefetcher:
    """``for _ in BatchPrefetcher(batches, targets): optimizer.step(closure)``.

    ``batches`` yields tuples of (pinned) host tensors, ``targets`` are the fixed device tensors the
    closure reads, one per element of a batch.  On each iteration the targets hold the next batch
    (the copy into them is ordered on the current stream) and the batch after it is already on its
    way.  Yields the index of the batch."""

    def __init__(self, batches: Iterable[Sequence[torch.Tensor]], targets: Sequence[torch.Tensor]):
        self._it = iter(batches)
        self._targets = list(targets)
        self._stream = torch.cuda.Stream(device=self._targets[0].device)
        self._stage = [[torch.empty_like(t) for t in self._targets] for _ in range(2)]
        self._ready = [torch.cuda.Event(), torch.cuda.Event()]
        self._free = [torch.cuda.Event(), torch.cuda.Event()]

    def _issue(self, slot: int) -> bool:
        try:
            batch = next(self._it)
        except StopIteration:
            return False
        self._stream.wait_event(self._free[slot])       # the step that last read this slot has taken its copy
        with torch.cuda.stream(self._stream):
            for dst, src in zip(self._stage[slot], batch):
                dst.copy_(src, non_blocking=True)
            self._ready[slot].record(self._stream)
        return True

    def __iter__(self):
        main = torch.cuda.current_stream(self._targets[0].device)
        for ev in self._free:
            ev.record(main)
        have = self._issue(0)
        i = 0
        while have:
            slot = i & 1
            main.wait_event(self._ready[slot])
            for dst, src in zip(self._targets, self._stage[slot]):
                dst.copy_(src, non_blocking=True)
            self._free[slot].record(main)
            have = self._issue(slot ^ 1)                # overlaps with the step the caller runs now
            yield i
            i += 1
