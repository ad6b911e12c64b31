"""Seeded synthetic extreme-classification workloads.

Text: token ids uniform in ``[token_lo, vocab)``, per-row length uniform in ``[len_lo, len_hi]``,
padded with id 0 (attention mask 0 there).  Targets: every row has ``1 + Poisson(lam)`` distinct
positive labels drawn without replacement from a Zipf(s) distribution over ``[0, L)``.

The generator is a pure function of ``(seed, row index)`` blocks, so every rank can materialise
the same global batch without communication — the property the reference gets from identical
DataLoader seeds on every rank (main.py:22-24, 101-122).
"""
from __future__ import annotations

from dataclasses import dataclass, asdict

import numpy as np
import scipy.sparse as sp


@dataclass(frozen=True)
class SyntheticSpec:
    num_labels: int
    seq_len: int = 32
    len_lo: int = 6
    len_hi: int = 32
    vocab: int = 30522
    token_lo: int = 1000
    poisson_lam: float = 1.3
    zipf_s: float = 1.1
    seed: int = 0

    def to_dict(self) -> dict:
        return asdict(self)


class ZipfSampler:
    """Inverse-CDF sampler for P(l) ∝ (l+1)^-s over ``[0, L)``.

    The CDF over up to 1e8 labels is not stored in full: ranks below ``head`` use an exact table,
    the tail uses the continuous approximation of the partial sums (Euler–Maclaurin), which is
    accurate to <1e-6 relative beyond the head.
    """

    def __init__(self, num_labels: int, s: float, head: int = 1 << 20):
        self.L = int(num_labels)
        self.s = float(s)
        self.head = int(min(head, self.L))
        w = np.power(np.arange(1, self.head + 1, dtype=np.float64), -self.s)
        self.head_cum = np.cumsum(w)
        self.head_mass = float(self.head_cum[-1])
        self.tail_mass = self._integral(self.head, self.L) if self.L > self.head else 0.0
        self.total = self.head_mass + self.tail_mass

    def _integral(self, a: float, b: float) -> float:
        # sum_{k=a+1}^{b} k^-s ≈ ∫_{a+1/2}^{b+1/2} x^-s dx  (midpoint rule)
        s = self.s
        lo, hi = a + 0.5, b + 0.5
        if abs(s - 1.0) < 1e-12:
            return float(np.log(hi / lo))
        return float((hi ** (1 - s) - lo ** (1 - s)) / (1 - s))

    def sample(self, rng: np.random.Generator, n: int) -> np.ndarray:
        u = rng.random(n) * self.total
        out = np.empty(n, dtype=np.int64)
        in_head = u < self.head_mass
        out[in_head] = np.searchsorted(self.head_cum, u[in_head], side="right")
        if (~in_head).any():
            s = self.s
            r = u[~in_head] - self.head_mass
            lo = self.head + 0.5
            if abs(s - 1.0) < 1e-12:
                x = lo * np.exp(r)
            else:
                x = np.power(lo ** (1 - s) + r * (1 - s), 1.0 / (1 - s))
            out[~in_head] = np.clip(np.floor(x + 0.5).astype(np.int64) - 1, self.head, self.L - 1)
        return np.minimum(out, self.L - 1)


class SyntheticXC:
    """Materialises blocks of rows of a synthetic dataset described by a :class:`SyntheticSpec`."""

    BLOCK = 4096  # rows generated per RNG stream; row r lives in block r // BLOCK

    def __init__(self, spec: SyntheticSpec):
        self.spec = spec
        self.zipf = ZipfSampler(spec.num_labels, spec.zipf_s)
        self._cache: dict[int, tuple] = {}

    def _block(self, blk: int):
        hit = self._cache.get(blk)
        if hit is not None:
            return hit
        sp_ = self.spec
        rng = np.random.default_rng([sp_.seed, blk])
        n = self.BLOCK
        lens = rng.integers(sp_.len_lo, sp_.len_hi + 1, size=n)
        ids = rng.integers(sp_.token_lo, sp_.vocab, size=(n, sp_.seq_len), dtype=np.int64)
        mask = (np.arange(sp_.seq_len)[None, :] < lens[:, None]).astype(np.int64)
        ids = ids * mask
        npos = 1 + rng.poisson(sp_.poisson_lam, size=n)
        npos = np.minimum(npos, sp_.num_labels)
        indptr = np.zeros(n + 1, dtype=np.int64)
        cols = []
        for r in range(n):
            need = int(npos[r])
            got = np.unique(self.zipf.sample(rng, need))
            while len(got) < need:  # redraw duplicates (sampling without replacement)
                got = np.unique(np.concatenate([got, self.zipf.sample(rng, need - len(got))]))
            cols.append(got[:need])
            indptr[r + 1] = indptr[r] + need
        cols = np.concatenate(cols) if cols else np.zeros(0, dtype=np.int64)
        out = (ids, mask, indptr, cols)
        if len(self._cache) > 64:
            self._cache.clear()
        self._cache[blk] = out
        return out

    def rows(self, row_ids: np.ndarray):
        """Return ``(input_ids [n,S] int64, attention_mask [n,S] int64, labels CSR [n, L])``."""
        row_ids = np.asarray(row_ids, dtype=np.int64)
        n = len(row_ids)
        S = self.spec.seq_len
        ids = np.empty((n, S), dtype=np.int64)
        mask = np.empty((n, S), dtype=np.int64)
        indptr = np.zeros(n + 1, dtype=np.int64)
        cols = []
        for i, r in enumerate(row_ids):
            b_ids, b_mask, b_ptr, b_cols = self._block(int(r) // self.BLOCK)
            j = int(r) % self.BLOCK
            ids[i] = b_ids[j]
            mask[i] = b_mask[j]
            c = b_cols[b_ptr[j]: b_ptr[j + 1]]
            cols.append(c)
            indptr[i + 1] = indptr[i] + len(c)
        cols = np.concatenate(cols) if cols else np.zeros(0, dtype=np.int64)
        labels = sp.csr_matrix((np.ones(len(cols), dtype=np.float32), cols, indptr),
                               shape=(n, self.spec.num_labels))
        return ids, mask, labels

    def batch(self, step: int, global_batch: int):
        """Global batch of step ``step`` (rows ``step*B .. step*B+B-1``)."""
        return self.rows(np.arange(step * global_batch, (step + 1) * global_batch))

    def materialise(self, num_rows: int):
        return self.rows(np.arange(num_rows))
