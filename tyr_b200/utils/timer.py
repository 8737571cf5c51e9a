"""Wall-clock and device timers, NVTX ranges (the reference times with `IO.monoMsNow` and CUDA events,
Tests/RunLagunaFused.lean:250-268)."""
from __future__ import annotations

import contextlib
import time
from typing import Dict, List, Optional

import torch


class Timer:
    """Named accumulating timers; ``sync`` waits for the device before reading the clock."""

    def __init__(self, sync: bool = False, device=None):
        self.sync, self.device = sync, device
        self.totals: Dict[str, float] = {}
        self.counts: Dict[str, int] = {}

    @contextlib.contextmanager
    def section(self, name: str):
        if self.sync and torch.cuda.is_available():
            torch.cuda.synchronize(self.device)
        t0 = time.perf_counter()
        try:
            yield
        finally:
            if self.sync and torch.cuda.is_available():
                torch.cuda.synchronize(self.device)
            self.totals[name] = self.totals.get(name, 0.0) + (time.perf_counter() - t0)
            self.counts[name] = self.counts.get(name, 0) + 1

    def mean_ms(self, name: str) -> float:
        return 1e3 * self.totals.get(name, 0.0) / max(1, self.counts.get(name, 0))

    def report(self) -> str:
        return "\n".join(f"{k}: {1e3 * v:.2f} ms total, {self.mean_ms(k):.3f} ms mean over {self.counts[k]}" for k, v in self.totals.items())


def time_cuda(fn, iters: int = 20, warmup: int = 3, flush_bytes: int = 0) -> float:
    """Median milliseconds per call, CUDA events on the current stream; optionally writes ``flush_bytes`` between
    iterations to evict L2."""
    flush = torch.empty(flush_bytes, dtype=torch.uint8, device="cuda") if flush_bytes else None
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    ts: List[float] = []
    for _ in range(iters):
        if flush is not None:
            flush.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1))
    return sorted(ts)[len(ts) // 2]


@contextlib.contextmanager
def nvtx_range(name: str):
    """NVTX range when CUDA is present (shows up in Nsight timelines); no-op otherwise."""
    on = torch.cuda.is_available()
    if on:
        torch.cuda.nvtx.range_push(name)
    try:
        yield
    finally:
        if on:
            torch.cuda.nvtx.range_pop()


def mono_ms() -> int:
    return int(time.monotonic() * 1000)
