"""Phase timing on the device: CUDA events around named regions of a step (wall clock on CPU).

``PhaseTimer`` is used by ``XCTrainer.profile_step`` to report where a step's time goes (encoder forward,
all-gather + classifier step, reduce-scatter, encoder backward, optimizer) without a profiler: events are
recorded on the launching stream and read after one synchronize, so the figures are device times, not host
times.  The reference has no timing beyond tqdm's iteration rate.
"""
from __future__ import annotations

import os
import time
from contextlib import contextmanager

import torch

_NVTX = os.environ.get("RENEE_B200_NVTX", "") == "1"


def nvtx_enabled() -> bool:
    return _NVTX and torch.cuda.is_available()


@contextmanager
def nvtx_range(name: str):
    """NVTX range around a phase of the step when ``RENEE_B200_NVTX=1`` (for timeline profilers; a no-op
    otherwise).  Ranges are host-side annotations: they label the launches of an eager step, and the capture —
    not the replays — of a CUDA-graph step, so profile with ``cuda_graph=False``."""
    if not nvtx_enabled():
        yield
        return
    torch.cuda.nvtx.range_push(name)
    try:
        yield
    finally:
        torch.cuda.nvtx.range_pop()


class PhaseTimer:
    def __init__(self, device):
        self.cuda = torch.device(device).type == "cuda"
        self.marks: list = []

    @contextmanager
    def phase(self, name: str):
        with nvtx_range(name):
            yield from self._phase(name)

    def _phase(self, name: str):
        if self.cuda:
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            yield
            b.record()
            self.marks.append((name, a, b))
        else:
            t0 = time.perf_counter()
            yield
            self.marks.append((name, t0, time.perf_counter()))

    def result_ms(self) -> dict:
        if self.cuda:
            torch.cuda.synchronize()
            out = {}
            for name, a, b in self.marks:
                out[name] = out.get(name, 0.0) + a.elapsed_time(b)
            return out
        out = {}
        for name, a, b in self.marks:
            out[name] = out.get(name, 0.0) + (b - a) * 1e3
        return out
