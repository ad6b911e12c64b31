import numpy as np
import scipy.sparse as sp


def compute_inv_propesity(labels, A, B):
    n = labels.shape[0]
    freq = np.asarray(labels.sum(axis=0)).ravel()
    C = (np.log(n) - 1) * (B + 1) ** A
    return 1.0 + C * np.power(freq + B, -A)


class Metrics:
    """P@k / nDCG@k (and propensity-scored variants) for a CSR score matrix."""

    def __init__(self, true_labels, inv_psp=None):
        self.true = sp.csr_matrix(true_labels).astype(np.float32)
        self.inv_psp = inv_psp

    def _topk(self, mat, k):
        mat = sp.csr_matrix(mat)
        out = np.full((mat.shape[0], k), -1, dtype=np.int64)
        for r in range(mat.shape[0]):
            lo, hi = mat.indptr[r], mat.indptr[r + 1]
            o = np.argsort(-mat.data[lo:hi], kind="stable")[:k]
            out[r, : len(o)] = mat.indices[lo:hi][o]
        return out

    def _eval(self, pred, w, k):
        n = pred.shape[0]
        hit = np.zeros((n, k))
        for r in range(n):
            t = set(self.true.indices[self.true.indptr[r]: self.true.indptr[r + 1]].tolist())
            for j, c in enumerate(pred[r]):
                if c in t:
                    hit[r, j] = 1.0 if w is None else w[c]
        prec = (np.cumsum(hit, 1) / np.arange(1, k + 1)).mean(0)
        disc = 1 / np.log2(np.arange(2, k + 2))
        ntrue = np.diff(self.true.indptr)
        dcg = np.cumsum(hit * disc, 1)
        cum = np.cumsum(disc)
        nd = np.zeros_like(dcg)
        for j in range(k):
            cnt = np.minimum(ntrue, j + 1)
            nd[:, j] = dcg[:, j] / np.where(cnt > 0, cum[np.maximum(cnt, 1) - 1], 1.0)
        return prec, nd.mean(0)

    def eval(self, score_mat, K=5):
        pred = self._topk(score_mat, K)
        p, n = self._eval(pred, None, K)
        if self.inv_psp is None:
            return [p, n]
        w = np.asarray(self.inv_psp).ravel()
        best = self._topk(self.true.multiply(w[None, : self.true.shape[1]]), K)
        pp, pn = self._eval(pred, w, K)
        bp, bn = self._eval(best, w, K)
        with np.errstate(divide="ignore", invalid="ignore"):
            return [p, n, np.nan_to_num(pp / bp), np.nan_to_num(pn / bn)]
