"""Batch collation for the hybrid data/model-parallel step, and the rank-coordinated sampler.

Every rank sees the SAME global batch of row ids.  A rank encodes only its own slice of rows but
needs the positives of ALL rows restricted to its own label shard (parity: reference ``XCCollator``
dl_base.py:900-978 and the seed-coordinated DataLoaders of main.py:101-122).

Differences from the reference, made for the fused kernels:

* positives are emitted as int32 ``(row in the GLOBAL batch, local_label)`` pairs **sorted by local
  label id** (ties by row), so a CTA that owns a 128-label tile finds its positives with two binary
  searches instead of a dense target or an ``index_put_`` pass.  The layout does not depend on
  ``--accum``: the classifier splits the step over the LABEL axis (``models/xfc.py``), every label
  chunk sees all rows of the batch, and a chunk's positives are a contiguous range of the sorted
  list.  (The reference splits the rows instead and rebases them per micro-batch,
  dl_base.py:939-959; that convention does not exist here.);
* duplicates are removed on the host (the reference's ``out[pos_x,pos_y] -= 1`` is a
  non-accumulating indexed write, dl_base.py:594);
* the sampler is a pure function of ``(seed, epoch)``, so ranks agree by construction rather than
  by running identically seeded worker processes.
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np
import scipy.sparse as sp
import torch

from ..utils.sharding import LabelSharding, batch_row_range


@dataclass
class XCBatch:
    batch_size: int                     # global rows in this step (B)
    numy: int                           # padded label count (Lp)
    input_ids: torch.Tensor             # [b_local, S] int32
    attention_mask: torch.Tensor        # [b_local, S] int32
    pos_rows: torch.Tensor | None = None      # [nnz] int32, row inside the global batch
    pos_labels: torch.Tensor | None = None    # [nnz] int32, label id inside this rank's shard (ascending)
    row_ids: np.ndarray | None = None   # global dataset rows (for evaluation bookkeeping)
    dense_targets: torch.Tensor | None = None  # [B, Ls] float (default/autograd path only)
    uploaded: object = None             # callable or None: the consumer calls it once its host-to-device copies of
                                        # this batch are issued (pinned staging slots of PrefetchLoader)

    @property
    def z(self) -> torch.Tensor:
        """``[2, nnz]`` int64 COO in the reference's batch-dict layout (dl_base.py:962-971)."""
        return torch.stack([self.pos_rows.long(), self.pos_labels.long()])

    def pin(self) -> "XCBatch":
        for name in ("input_ids", "attention_mask", "pos_rows", "pos_labels"):
            t = getattr(self, name)
            if isinstance(t, torch.Tensor) and not t.is_pinned() and torch.cuda.is_available():
                setattr(self, name, t.pin_memory())
        return self


class XCCollator:
    """``accum`` and ``xfc_batch`` keep the reference collator's argument list (dl_base.py:900-912); they
    do not change what is emitted (see the module docstring)."""

    def __init__(self, sharding: LabelSharding, dataset, rank: int, accum: int = 1, xfc_batch: int = 0,
                 train: bool = True, dense_targets: bool = False):
        self.sharding = sharding
        self.dataset = dataset
        self.rank = rank
        self.world_size = sharding.world_size
        self.accum = accum
        self.xfc_batch = xfc_batch
        self.train = train
        self.dense_targets = dense_targets
        self.lo, self.hi = sharding.shard_range(rank)
        self._shard_labels = None

    def _labels(self) -> sp.csr_matrix:
        if self._shard_labels is None:
            lab = self.dataset.labels.tocsc()
            hi = min(self.hi, lab.shape[1])
            lo = min(self.lo, hi)
            self._shard_labels = lab[:, lo:hi].tocsr()
            self._shard_labels.sum_duplicates()
        return self._shard_labels

    def __call__(self, row_ids) -> XCBatch:
        full_ids = np.asarray(row_ids, dtype=np.int64)
        bsz = len(full_ids)
        s, e = batch_row_range(bsz, self.world_size, self.rank)
        ids, mask = self.dataset.get_fts(full_ids[s:e])
        batch = XCBatch(batch_size=bsz, numy=self.sharding.padded_labels,
                        input_ids=torch.from_numpy(np.ascontiguousarray(ids, dtype=np.int32)),
                        attention_mask=torch.from_numpy(np.ascontiguousarray(mask, dtype=np.int32)),
                        row_ids=full_ids)
        if not self.train:
            return batch
        coo = self._labels()[full_ids].tocoo()
        rows = coo.row.astype(np.int64)
        cols = coo.col.astype(np.int64)
        keep = coo.data != 0
        rows, cols = rows[keep], cols[keep]
        order = np.lexsort((rows, cols))
        rows, cols = rows[order], cols[order]
        batch.pos_rows = torch.from_numpy(rows.astype(np.int32))
        batch.pos_labels = torch.from_numpy(cols.astype(np.int32))
        if self.dense_targets:
            y = torch.zeros(bsz, self.sharding.labels_per_rank)
            y[torch.from_numpy(coo.row[keep].astype(np.int64)), torch.from_numpy(coo.col[keep].astype(np.int64))] = 1.0
            batch.dense_targets = y
        return batch


class GlobalBatchSampler:
    """Yields the same sequence of global batches of row ids on every rank.

    ``shuffle=True`` draws one permutation per epoch from ``default_rng([seed, epoch])``.  The last
    batch of an epoch may be partial (kept, like ``drop_last=False`` in the reference loaders)."""

    def __init__(self, num_points: int, global_batch: int, shuffle: bool, seed: int):
        self.num_points = int(num_points)
        self.global_batch = int(global_batch)
        self.shuffle = shuffle
        self.seed = int(seed)

    def __len__(self) -> int:
        return (self.num_points + self.global_batch - 1) // self.global_batch

    def epoch(self, epoch: int):
        if self.shuffle:
            perm = np.random.default_rng([self.seed, epoch]).permutation(self.num_points)
        else:
            perm = np.arange(self.num_points)
        for s in range(0, self.num_points, self.global_batch):
            yield perm[s: s + self.global_batch]


class _StagingSlot:
    """One set of page-locked host buffers that successive batches are copied into.  Allocating page-locked
    memory per batch goes through the driver (and, once the consumer runs ahead of the device, cannot be served from
    a cache, because the previous blocks are still being read by queued copies); a fixed ring is allocated once.
    A slot is refilled only after the copies issued from its previous batch have completed: the consumer records
    an event behind them (``XCBatch.uploaded``), the loader thread waits for it.  A consumer that never calls
    ``uploaded`` costs a device synchronisation at reuse instead."""

    NAMES = ("input_ids", "attention_mask", "pos_rows", "pos_labels")

    def __init__(self):
        self.bufs: dict = {}
        self.event = None
        self.handed_out = False

    def _buffer(self, name: str, t: torch.Tensor) -> torch.Tensor:
        buf = self.bufs.get(name)
        n = t.numel()
        if buf is None or buf.numel() < n or buf.dtype != t.dtype:
            buf = torch.empty(max(n + n // 4, 64), dtype=t.dtype)
            if torch.cuda.is_available():
                buf = buf.pin_memory()
            self.bufs[name] = buf
        return buf[:n].view(t.shape)

    def wait(self) -> None:
        if not self.handed_out:
            return
        if self.event is not None:
            self.event.synchronize()
        elif torch.cuda.is_available():
            torch.cuda.synchronize()
        self.handed_out, self.event = False, None

    def mark_uploaded(self) -> None:
        if torch.cuda.is_available():
            ev = torch.cuda.Event()
            ev.record()
            self.event = ev

    def fill(self, b: XCBatch) -> XCBatch:
        for name in self.NAMES:
            t = getattr(b, name)
            if isinstance(t, torch.Tensor):
                v = self._buffer(name, t)
                v.copy_(t)
                setattr(b, name, v)
        b.uploaded = self.mark_uploaded
        self.handed_out = True
        return b


class PrefetchLoader:
    """Background-thread loader: collates the next batches while the device runs the current step.
    (The reference uses 4 DataLoader worker processes, main.py:102; collation here is a handful of
    numpy gathers, so one thread and a ring of pinned staging buffers are enough.)"""

    def __init__(self, sampler: GlobalBatchSampler, collator: XCCollator, depth: int = 3, pin: bool = False):
        self.sampler = sampler
        self.collator = collator
        self.depth = depth
        self.pin = pin
        # a batch can be in the queue (depth), in the consumer's hands (1) or being filled (1)
        self._slots = [_StagingSlot() for _ in range(depth + 2)] if pin else []
        self._next_slot = 0

    def __len__(self) -> int:
        return len(self.sampler)

    @property
    def dataset(self):
        return self.collator.dataset

    def epoch(self, epoch: int):
        import queue
        import threading

        q: "queue.Queue" = queue.Queue(maxsize=self.depth)
        stop = threading.Event()

        def work():
            try:
                for ids in self.sampler.epoch(epoch):
                    if stop.is_set():
                        return
                    b = self.collator(ids)
                    if self.pin:
                        slot = self._slots[self._next_slot]
                        self._next_slot = (self._next_slot + 1) % len(self._slots)
                        slot.wait()
                        b = slot.fill(b)
                    q.put(b)
                q.put(None)
            except BaseException as exc:  # surfaced to the consumer
                q.put(exc)

        t = threading.Thread(target=work, daemon=True)
        t.start()
        try:
            while True:
                item = q.get()
                if item is None:
                    break
                if isinstance(item, BaseException):
                    raise item
                yield item
        finally:
            stop.set()
            while not q.empty():
                try:
                    q.get_nowait()
                except Exception:
                    break
