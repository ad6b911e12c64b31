"""Host-side failure detection: store-based heartbeats and an abort-before-launch check.

The reference has no failure handling beyond NCCL's default timeouts (a dead rank stalls the others
until the collective times out).  With collectives fused into kernels that wait on peer flags, a dead
peer must be noticed on the HOST, before kernels that would wait for it are launched:

* every rank runs a :class:`Heartbeat` thread that stamps ``hb/<rank>`` in a ``torch.distributed``
  store (TCPStore / FileStore / HashStore) every ``interval`` seconds;
* the same thread reads the peers' stamps and the failure key once per interval (``poll``) and keeps the
  verdict in a local field;
* ``check()`` — called by the trainer before each step's launches — raises :class:`PeerFailure` if that
  verdict says a peer's stamp is older than ``timeout`` or a rank has posted a failure with
  ``post_failure``.  With the thread running it touches no store: a step of a millisecond must not pay
  a dozen TCP round trips.  Without a thread (manual driving in tests) it polls the store itself;
* the device-side waits are bounded anyway (they return a status word instead of hanging), so a
  failure that slips between two checks costs one timed-out step, not a hung GPU.

Recovery is restart-from-checkpoint (``--checkpoint-resume``), as in the reference.
"""
from __future__ import annotations

import threading
import time


class PeerFailure(RuntimeError):
    def __init__(self, msg: str, ranks: list[int]):
        super().__init__(msg)
        self.ranks = ranks


class Heartbeat:
    def __init__(self, store, rank: int, world_size: int, interval: float = 1.0, timeout: float = 10.0,
                 clock=time.time):
        self.store = store
        self.rank = rank
        self.world = world_size
        self.interval = float(interval)
        self.timeout = float(timeout)
        self.clock = clock
        self._stop = threading.Event()
        self._thread = None
        self._start_time = clock()
        self._failure: PeerFailure | None = None     # written by the thread, read by check()

    def _key(self, r: int) -> str:
        return f"hb/{r}"

    def beat(self) -> None:
        self.store.set(self._key(self.rank), repr(self.clock()))

    def start(self) -> "Heartbeat":
        self.beat()

        def loop():
            while not self._stop.wait(self.interval):
                try:
                    self.beat()
                    f = self.poll()
                except Exception:
                    return
                if f is not None:
                    self._failure = f

        self._thread = threading.Thread(target=loop, daemon=True, name=f"heartbeat-{self.rank}")
        self._thread.start()
        return self

    def stop(self) -> None:
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2 * self.interval + 1)

    def post_failure(self, message: str) -> None:
        self.store.set("failure", f"{self.rank}:{message}")

    def _get(self, key: str):
        try:
            if hasattr(self.store, "check") and not self.store.check([key]):
                return None
            return self.store.get(key).decode()
        except Exception:
            return None

    def stale_peers(self) -> list[int]:
        now = self.clock()
        bad = []
        for r in range(self.world):
            if r == self.rank:
                continue
            v = self._get(self._key(r))
            last = float(v) if v is not None else self._start_time
            if now - last > self.timeout:
                bad.append(r)
        return bad

    def poll(self) -> PeerFailure | None:
        """Reads the failure key and every peer's stamp from the store (blocking round trips)."""
        f = self._get("failure")
        if f is not None:
            r, _, msg = f.partition(":")
            return PeerFailure(f"rank {r} reported a failure: {msg}", [int(r)])
        bad = self.stale_peers()
        if bad:
            return PeerFailure(f"no heartbeat from rank(s) {bad} for more than {self.timeout:.1f} s", bad)
        return None

    def check(self) -> None:
        """Step-path check: a field read while the heartbeat thread runs, a direct ``poll`` otherwise."""
        running = self._thread is not None and self._thread.is_alive() and not self._stop.is_set()
        f = self._failure if running else (self._failure or self.poll())
        if f is not None:
            raise f
