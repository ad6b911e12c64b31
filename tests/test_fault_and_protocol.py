"""Peer-memory protocol on CPU threads (fake backend) and host-side failure detection.

No GPU is involved and nothing is made to fault: failures are a rank that never joins, a rank that stops
beating, and a posted error."""
import threading
import time

import numpy as np
import pytest
import torch.distributed as dist

from renee_b200.parallel.fake_peer import STATUS_OK, STATUS_TIMEOUT, FakePeerRank, FakePeerWorld
from renee_b200.parallel.watchdog import Heartbeat, PeerFailure
from renee_b200.utils.sharding import batch_row_range


def _rank_loop(world, r, steps, rows_of, partial_of, grad_of, out, jitter):
    k = FakePeerRank(world, r, wait_budget_s=5.0)
    rng = np.random.default_rng(r)
    res = []
    for t in range(1, steps + 1):
        k.begin_step()
        if jitter:
            time.sleep(float(rng.random()) * 0.003)
        k.ag_push(rows_of(r, t))
        X = k.ag_wait().copy()
        if jitter:
            time.sleep(float(rng.random()) * 0.003)
        k.rs_publish(partial_of(r, t, X))
        dx = k.rs_pull()
        g = k.grad_allreduce(grad_of(r, t))
        res.append((X, dx, g))
    out[r] = (k.status, res)


@pytest.mark.parametrize("G,B", [(2, 8), (4, 10), (8, 16)])
def test_protocol_matches_collective_semantics_under_interleavings(G, B):
    D, n_grad, steps = 4, 37, 12
    world = FakePeerWorld(G, B, D, n_grad)

    def rows_of(r, t):
        s, e = batch_row_range(B, G, r)
        return np.arange((e - s) * D, dtype=np.float32).reshape(e - s, D) + 100 * r + 1000 * t

    def partial_of(r, t, X):
        return X * (r + 1) + t

    def grad_of(r, t):
        return np.arange(n_grad, dtype=np.float32) * (r + 1) + t

    out = {}
    threads = [threading.Thread(target=_rank_loop, args=(world, r, steps, rows_of, partial_of, grad_of, out, True))
               for r in range(G)]
    [t.start() for t in threads]
    [t.join() for t in threads]
    for r in range(G):
        status, res = out[r]
        assert status == STATUS_OK
        for t, (X, dx, g) in enumerate(res, start=1):
            X_want = np.concatenate([rows_of(q, t) for q in range(G)])
            np.testing.assert_array_equal(X, X_want)
            s, e = batch_row_range(B, G, r)
            np.testing.assert_allclose(dx, sum(partial_of(q, t, X_want) for q in range(G))[s:e])
            np.testing.assert_allclose(g, sum(grad_of(q, t) for q in range(G)))


def test_missing_rank_times_out_with_status_instead_of_hanging():
    G, B, D = 3, 6, 2
    world = FakePeerWorld(G, B, D, 8)
    out = {}

    def loop(r):
        k = FakePeerRank(world, r, wait_budget_s=0.3)
        k.begin_step()
        k.ag_push(np.ones((2, D), dtype=np.float32))
        X = k.ag_wait()
        out[r] = (k.status, k.status_detail, X)

    threads = [threading.Thread(target=loop, args=(r,)) for r in (0, 1)]    # rank 2 never joins
    t0 = time.monotonic()
    [t.start() for t in threads]
    [t.join() for t in threads]
    assert time.monotonic() - t0 < 5.0
    for r in (0, 1):
        status, detail, X = out[r]
        assert status == STATUS_TIMEOUT and detail == ("all-gather", [2]) and X is None


def test_heartbeat_detects_silent_and_reported_failures():
    store = dist.HashStore()
    now = [100.0]
    hb = [Heartbeat(store, r, 3, interval=0.05, timeout=5.0, clock=lambda: now[0]) for r in range(3)]
    for h in hb:
        h.beat()
    hb[0].check()                              # everyone fresh
    now[0] += 4.0
    hb[1].beat()                               # rank 1 keeps beating, rank 2 went silent
    now[0] += 2.0
    with pytest.raises(PeerFailure) as ei:
        hb[0].check()
    assert ei.value.ranks == [2]
    hb[2].beat()
    hb[0].check()
    hb[1].post_failure("CUDA error: peer wait timed out")
    with pytest.raises(PeerFailure, match="rank 1 reported"):
        hb[0].check()


def test_heartbeat_thread_runs_and_stops():
    store = dist.HashStore()
    a = Heartbeat(store, 0, 2, interval=0.02, timeout=0.5).start()
    b = Heartbeat(store, 1, 2, interval=0.02, timeout=0.5).start()
    time.sleep(0.1)
    a.check(); b.check()
    b.stop()                                    # rank 1 "dies" between steps
    time.sleep(0.7)
    with pytest.raises(PeerFailure):
        a.check()
    a.stop()


def test_check_reads_no_store_while_the_thread_runs():
    """A step of a millisecond cannot afford store round trips: with the thread alive, ``check`` is a field read."""
    class Counting:
        def __init__(self):
            self.inner, self.calls = dist.HashStore(), 0

        def set(self, k, v):
            self.inner.set(k, v)

        def check(self, keys):
            self.calls += 1
            return self.inner.check(keys)

        def get(self, k):
            self.calls += 1
            return self.inner.get(k)

    store = Counting()
    a = Heartbeat(store, 0, 2, interval=0.05, timeout=0.3).start()
    b = Heartbeat(store, 1, 2, interval=0.05, timeout=0.3).start()
    time.sleep(0.12)
    main_thread_calls = []
    orig_check, orig_get = store.check, store.get
    me = threading.get_ident()
    store.check = lambda keys: (main_thread_calls.append(1) if threading.get_ident() == me else None, orig_check(keys))[1]
    store.get = lambda k: (main_thread_calls.append(1) if threading.get_ident() == me else None, orig_get(k))[1]
    for _ in range(1000):
        a.check()
    assert not main_thread_calls
    b.stop()
    time.sleep(0.6)                             # the thread of rank 0 notices within timeout + interval
    with pytest.raises(PeerFailure):
        a.check()
    assert not main_thread_calls
    a.stop()
