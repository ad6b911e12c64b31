"""Extreme-classification metrics: P@k, nDCG@k and their propensity-scored variants.

The reference delegates these to pyxclib (``xclib.evaluation.xc_metrics``; call sites
dl_base.py:41-54 ``printacc`` and main.py:57-60 ``compute_inv_propesity``).  pyxclib is an external
package, so the formulas are implemented here from their published definitions
(Jain et al., "Extreme multi-label loss functions ...", KDD 2016):

* inverse propensity of label ``l`` with train frequency ``n_l`` over ``N`` points:
  ``1 + C (n_l + B)^-A`` with ``C = (log N - 1)(B + 1)^A``;
* ``P@k   = mean_rows( (1/k) sum_{i<=k} hit_i )``;
* ``nDCG@k = mean_rows( sum_{i<=k} hit_i/log2(i+1) / sum_{i<=min(k,|y|)} 1/log2(i+1) )``;
* ``PSP@k``/``PSnDCG@k`` weight each hit by the label's inverse propensity and divide by the value
  reached by the best possible ranking (true labels sorted by inverse propensity).

All values are returned as percentages in a table whose rows are ``P, nDCG, PSP, PSnDCG`` and whose
columns are ``1..K`` — the layout the reference writes to ``evaluation.tsv`` (dl_base.py:833-839).
"""
from __future__ import annotations

import numpy as np
import scipy.sparse as sp

METRIC_NAMES = ("P", "nDCG", "PSP", "PSnDCG")


def propensity_constants(dataset_name: str) -> tuple[float, float]:
    """(A, B) picked from the dataset folder name (reference main.py:57-59)."""
    if "Amazon" in dataset_name:
        return 0.6, 2.6
    if "Wiki" in dataset_name:
        return 0.5, 0.4
    return 0.55, 1.5


def compute_inv_propensity(trn_labels: sp.spmatrix, A: float, B: float) -> np.ndarray:
    n_points = trn_labels.shape[0]
    freq = np.asarray((trn_labels != 0).sum(axis=0)).ravel().astype(np.float64)
    C = (np.log(n_points) - 1.0) * (B + 1.0) ** A
    return 1.0 + C * np.power(freq + B, -A)


def topk_indices(score_mat: sp.csr_matrix, k: int, pad: int = -1) -> np.ndarray:
    """Column ids of the ``k`` largest stored scores of each row (descending); rows with fewer
    than ``k`` stored entries are padded with ``pad``.  Ties keep the lower column first."""
    score_mat = score_mat.tocsr()
    n = score_mat.shape[0]
    out = np.full((n, k), pad, dtype=np.int64)
    indptr, indices, data = score_mat.indptr, score_mat.indices, score_mat.data
    counts = np.diff(indptr)
    if len(data) and counts.min() == counts.max() and counts[0] > 0:
        # regular layout (the predictor emits exactly K entries per row): vectorised path
        c = int(counts[0])
        d = data.reshape(n, c)
        idx = indices.reshape(n, c)
        order = np.argsort(-d, axis=1, kind="stable")[:, :k]
        kk = order.shape[1]
        out[:, :kk] = np.take_along_axis(idx, order, axis=1)
        return out
    for r in range(n):
        lo, hi = indptr[r], indptr[r + 1]
        if hi == lo:
            continue
        order = np.argsort(-data[lo:hi], kind="stable")[:k]
        out[r, : len(order)] = indices[lo:hi][order]
    return out


def _hits(pred: np.ndarray, true: sp.csr_matrix, weights: np.ndarray | None) -> np.ndarray:
    """hit[r, i] = (weight of pred[r, i]) if it is a true label of row r else 0."""
    n, k = pred.shape
    true = true.tocsr()
    L = true.shape[1]
    valid = (pred >= 0) & (pred < L)
    rows = np.repeat(np.arange(n), k).reshape(n, k)
    safe = np.where(valid, pred, 0)
    vals = np.asarray(true[rows.ravel(), safe.ravel()]).reshape(n, k)
    hit = ((vals != 0) & valid).astype(np.float64)
    if weights is not None:
        hit = hit * weights[safe]
    return hit


def _precision(hit: np.ndarray) -> np.ndarray:
    k = hit.shape[1]
    return (np.cumsum(hit, axis=1) / np.arange(1, k + 1)).mean(axis=0)


def _ndcg(hit: np.ndarray, n_true: np.ndarray) -> np.ndarray:
    k = hit.shape[1]
    disc = 1.0 / np.log2(np.arange(2, k + 2))
    dcg = np.cumsum(hit * disc, axis=1)
    cum = np.cumsum(disc)
    out = np.empty_like(dcg)
    for j in range(k):
        cnt = np.minimum(n_true, j + 1)
        den = np.where(cnt > 0, cum[np.maximum(cnt, 1) - 1], 1.0)
        out[:, j] = dcg[:, j] / den
    return out.mean(axis=0)


class Metrics:
    """``Metrics(true_labels, inv_psp).eval(score_mat, K)`` → ``[P, nDCG, PSP, PSnDCG]`` arrays of
    length K (fractions, not percentages), mirroring the pyxclib object used at dl_base.py:45-46."""

    def __init__(self, true_labels: sp.spmatrix, inv_psp: np.ndarray | None = None):
        self.true = (true_labels.tocsr() != 0).astype(np.float32).tocsr()
        self.inv_psp = None if inv_psp is None else np.asarray(inv_psp, dtype=np.float64).ravel()
        self.n_true = np.asarray(self.true.sum(axis=1)).ravel().astype(np.int64)

    def eval(self, score_mat: sp.spmatrix, K: int = 5) -> list[np.ndarray]:
        pred = topk_indices(sp.csr_matrix(score_mat), K)
        hit = _hits(pred, self.true, None)
        res = [_precision(hit), _ndcg(hit, self.n_true)]
        if self.inv_psp is not None:
            w = self.inv_psp
            if len(w) < self.true.shape[1]:
                w = np.concatenate([w, np.ones(self.true.shape[1] - len(w))])
            whit = _hits(pred, self.true, w)
            best = topk_indices(self.true.multiply(w[None, : self.true.shape[1]]).tocsr(), K)
            bhit = _hits(best, self.true, w)
            with np.errstate(divide="ignore", invalid="ignore"):
                psp = np.nan_to_num(_precision(whit) / _precision(bhit))
                psn = np.nan_to_num(_ndcg(whit, self.n_true) / _ndcg(bhit, self.n_true))
            res += [psp, psn]
        return res


def filter_predictions(score_mat: sp.spmatrix, filter_mat: sp.spmatrix | None) -> sp.csr_matrix:
    """Zero the (row, col) pairs listed in ``filter_mat`` (reciprocal pairs of the test set) and
    drop them from the sparsity pattern (reference dl_base.py:56-67)."""
    score_mat = sp.csr_matrix(score_mat)
    if filter_mat is None:
        return score_mat
    pattern = (sp.csr_matrix(filter_mat) != 0).astype(score_mat.dtype)
    out = sp.csr_matrix(score_mat - score_mat.multiply(pattern))
    out.eliminate_zeros()
    return out


def metrics_table(score_mat: sp.spmatrix, true_labels: sp.spmatrix, inv_psp: np.ndarray | None, K: int = 5):
    """Percent table: rows ``P, nDCG[, PSP, PSnDCG]``, columns ``'1'..'K'`` (a pandas DataFrame,
    like ``printacc`` at dl_base.py:41-54)."""
    import pandas as pd

    vals = np.array(Metrics(true_labels, inv_psp).eval(score_mat, K)) * 100.0
    df = pd.DataFrame(vals)
    df.index = list(METRIC_NAMES[: len(vals)])
    df.columns = [str(i + 1) for i in range(K)]
    return df
