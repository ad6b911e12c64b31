"""Phase timing on the device: CUDA events around named regions of a step (wall clock on CPU).

``PhaseTimer`` is used by ``XCTrainer.profile_step`` to report where a step's time goes (encoder forward,
all-gather + classifier step, reduce-scatter, encoder backward, optimizer) without a profiler: events are
recorded on the launching stream and read after one synchronize, so the figures are device times, not host
times.  The reference has no timing beyond tqdm's iteration rate.
"""
from __future__ import annotations

import time
from contextlib import contextmanager

import torch


class PhaseTimer:
    def __init__(self, device):
        self.cuda = torch.device(device).type == "cuda"
        self.marks: list = []

    @contextmanager
    def phase(self, name: str):
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
