"""Phase timers and profiler ranges.

The reference wraps compute_gradients / apply_gradients in a ``record_function`` stub that returns a null context
(gpu_process_worker.py:49-51, 1280, 1349) and times phases with ``time.time()``. Here ``record_function`` opens an
NVTX range when CUDA is present, ``PhaseTimer`` measures phases on the device with CUDA events (no host sync until
``summary()``), and ``profile_window`` switches an opt-in ``torch.profiler`` trace on for a few steps.
"""
from __future__ import annotations

import contextlib
import time
from collections import defaultdict
from typing import Dict, Iterator, List, Optional, Tuple

import torch


@contextlib.contextmanager
def record_function(name: str) -> Iterator[None]:
    use = torch.cuda.is_available()
    if use:
        torch.cuda.nvtx.range_push(name)
    try:
        yield
    finally:
        if use:
            torch.cuda.nvtx.range_pop()


class PhaseTimer:
    """``with timer.phase("fwd"):`` records a CUDA-event pair on the current stream (wall clock on CPU)."""

    def __init__(self, enabled: bool = True, cuda: Optional[bool] = None):
        self.enabled = enabled
        self._pairs: Dict[str, List[Tuple[torch.cuda.Event, torch.cuda.Event]]] = defaultdict(list)
        self._wall: Dict[str, float] = defaultdict(float)
        self.cuda = torch.cuda.is_available() if cuda is None else bool(cuda)

    @contextlib.contextmanager
    def phase(self, name: str) -> Iterator[None]:
        if not self.enabled:
            yield
            return
        if self.cuda:
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            try:
                with record_function(name):
                    yield
            finally:
                b.record()
                self._pairs[name].append((a, b))
        else:
            t0 = time.time()
            try:
                yield
            finally:
                self._wall[name] += (time.time() - t0) * 1000.0

    def summary(self, reset: bool = True) -> Dict[str, float]:
        """Milliseconds per phase. Waits for the recorded events of this timer only (other roles' streams on the same GPU
        keep running)."""
        out: Dict[str, float] = dict(self._wall)
        if self.cuda and self._pairs:
            for name, pairs in self._pairs.items():
                pairs[-1][1].synchronize()
                out[name] = out.get(name, 0.0) + sum(a.elapsed_time(b) for a, b in pairs)
        if reset:
            self._pairs.clear()
            self._wall.clear()
        return out


@contextlib.contextmanager
def profile_window(path: Optional[str], active: bool = True) -> Iterator[None]:
    """Opt-in torch.profiler trace written to ``path`` (Chrome trace)."""
    if not path or not active:
        yield
        return
    acts = [torch.profiler.ProfilerActivity.CPU]
    if torch.cuda.is_available():
        acts.append(torch.profiler.ProfilerActivity.CUDA)
    with torch.profiler.profile(activities=acts) as prof:
        yield
    prof.export_chrome_trace(path)
