"""CPU stand-in for the peer-memory backend: the same flag / parity protocol over shared host arrays.

The GPU kernels of ``ops/csrc/comm.cu`` and the fused GEMM prologue/epilogue synchronise through
step-tagged flags in a symmetric heap and double-buffer everything a peer writes.  This module runs that
protocol with one Python thread per rank over numpy arrays, so that its logic — tags, parity, who
writes which slot, bounded waits that return a status instead of hanging — can be exercised under
arbitrary thread interleavings and with injected failures, without a GPU.

A "rank" here performs, per step: push its rows into every rank's X[parity] + raise AG flags; wait for
all AG flags; compute a partial dX into its own dXp[parity]; raise RS flags on every rank; wait for all RS
flags and pull the sum of its rows; signal / two-shot all-reduce / wait on a gradient vector.
"""
from __future__ import annotations

import threading
import time

import numpy as np

from ..utils.sharding import batch_row_range

F_AG, F_RS, F_ARA, F_ARB = 0, 16, 32, 48
STATUS_OK, STATUS_TIMEOUT = 0, 1004


class FakePeerWorld:
    def __init__(self, G: int, B: int, D: int, n_grad: int):
        self.G, self.B, self.D, self.n_grad = G, B, D, n_grad
        self.flags = [np.zeros(64, dtype=np.uint32) for _ in range(G)]
        self.X = [[np.zeros((B, D), dtype=np.float32) for _ in range(2)] for _ in range(G)]
        self.dXp = [[np.zeros((B, D), dtype=np.float32) for _ in range(2)] for _ in range(G)]
        self.grad = [np.zeros(n_grad, dtype=np.float32) for _ in range(G)]
        self.lock = threading.Lock()   # stands in for the release/acquire ordering of flag accesses


class FakePeerRank:
    def __init__(self, world: FakePeerWorld, rank: int, wait_budget_s: float = 2.0):
        self.w, self.rank, self.G = world, rank, world.G
        self.step = 0
        self.budget = wait_budget_s
        self.status = STATUS_OK
        self.status_detail = None

    @property
    def parity(self) -> int:
        return self.step & 1

    def begin_step(self) -> None:
        self.step += 1

    # -- signalling ------------------------------------------------------------------------
    def _set_flag(self, peer: int, index: int, value: int) -> None:
        with self.w.lock:
            self.w.flags[peer][index] = value

    def _wait_flags(self, base: int, want: int, what: str) -> bool:
        if self.status != STATUS_OK:
            return False
        t0 = time.monotonic()
        while True:
            with self.w.lock:
                vals = self.w.flags[self.rank][base: base + self.G].astype(np.int64)
            if ((vals - want) >= 0).all():
                return True
            if time.monotonic() - t0 > self.budget:
                self.status = STATUS_TIMEOUT
                self.status_detail = (what, [int(q) for q in np.nonzero((vals - want) < 0)[0]])
                return False
            time.sleep(0)

    # -- all-gather --------------------------------------------------------------------------
    def ag_push(self, rows: np.ndarray) -> None:
        s, e = batch_row_range(self.w.B, self.G, self.rank)
        for q in range(self.G):
            self.w.X[q][self.parity][s:e] = rows
            self._set_flag(q, F_AG + self.rank, self.step)

    def ag_wait(self):
        ok = self._wait_flags(F_AG, self.step, "all-gather")
        return self.w.X[self.rank][self.parity] if ok else None

    # -- reduce-scatter ----------------------------------------------------------------------
    def rs_publish(self, partial: np.ndarray) -> None:
        self.w.dXp[self.rank][self.parity][:] = partial
        for q in range(self.G):
            self._set_flag(q, F_RS + self.rank, self.step)

    def rs_pull(self):
        s, e = batch_row_range(self.w.B, self.G, self.rank)
        if not self._wait_flags(F_RS, self.step, "reduce-scatter"):
            return np.zeros((e - s, self.w.D), dtype=np.float32)
        return sum(self.w.dXp[q][self.parity][s:e] for q in range(self.G))

    # -- gradient all-reduce (two-shot) -------------------------------------------------------
    def grad_allreduce(self, g: np.ndarray) -> np.ndarray | None:
        self.w.grad[self.rank][:] = g
        for q in range(self.G):
            self._set_flag(q, F_ARA + self.rank, self.step)
        if not self._wait_flags(F_ARA, self.step, "grad-arrive"):
            return None
        n = self.w.n_grad
        per = (n + self.G - 1) // self.G
        lo, hi = min(n, per * self.rank), min(n, per * (self.rank + 1))
        total = sum(self.w.grad[q][lo:hi].copy() for q in range(self.G))
        for q in range(self.G):
            self.w.grad[q][lo:hi] = total
            self._set_flag(q, F_ARB + self.rank, self.step)
        if not self._wait_flags(F_ARB, self.step, "grad-done"):
            return None
        return self.w.grad[self.rank].copy()
