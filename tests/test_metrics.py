"""P/nDCG/PSP/PSnDCG@k against hand-computed values; filter semantics (reference dl_base.py:41-67)."""
import numpy as np
import scipy.sparse as sp

from renee_b200.utils.metrics import (Metrics, compute_inv_propensity, filter_predictions, metrics_table,
                                      propensity_constants, topk_indices)


def _case():
    true = sp.csr_matrix(np.array([[1, 0, 1, 0, 0, 0], [0, 1, 0, 0, 0, 0], [0, 0, 0, 0, 0, 0]], dtype=np.float32))
    score = sp.csr_matrix(np.array([[0.9, 0.8, 0.1, 0, 0, 0], [0.2, 0.1, 0.7, 0, 0, 0], [0.5, 0.4, 0.3, 0, 0, 0]], dtype=np.float32))
    return true, score


def test_precision_and_ndcg():
    true, score = _case()
    P, N = Metrics(true).eval(score, 3)
    # row0 hits [1,0,1]; row1 ranking (2,0,1) hits [0,0,1]; row2 none
    np.testing.assert_allclose(P, [(1 + 0 + 0) / 3, (0.5 + 0 + 0) / 3, (2 / 3 + 1 / 3 + 0) / 3], rtol=1e-6)
    d = 1 / np.log2(np.arange(2, 5))
    r0 = [1.0, d[0] / (d[0] + d[1]), (d[0] + d[2]) / (d[0] + d[1])]
    r1 = [0.0, 0.0, d[2] / d[0]]
    np.testing.assert_allclose(N, [(r0[i] + r1[i]) / 3 for i in range(3)], rtol=1e-6)


def test_propensity_scored():
    true, score = _case()
    w = np.array([2.0, 1.0, 4.0, 1.0, 1.0, 1.0])
    P, N, PSP, PSN = Metrics(true, w).eval(score, 2)
    # numerator@1: row0 hit label0 → 2 ; row1 miss ; row2 miss → mean 2/3
    # best@1: row0 best label2 → 4 ; row1 label1 → 1 ; row2 none → mean 5/3
    np.testing.assert_allclose(PSP[0], (2 / 3) / (5 / 3), rtol=1e-6)
    assert 0 < PSN[1] <= 1


def test_inv_propensity_formula():
    X = sp.csr_matrix(np.array([[1, 0], [1, 1], [1, 0], [0, 0]], dtype=np.float32))
    A, B = propensity_constants("LF-AmazonTitles-131K")
    assert (A, B) == (0.6, 2.6) and propensity_constants("LF-Wikipedia-500K") == (0.5, 0.4)
    assert propensity_constants("other") == (0.55, 1.5)
    inv = compute_inv_propensity(X, A, B)
    C = (np.log(4) - 1) * (B + 1) ** A
    np.testing.assert_allclose(inv, 1 + C * (np.array([3, 1]) + B) ** -A)


def test_filter_and_topk_and_table():
    true, score = _case()
    filt = sp.csr_matrix(([1.0], ([0], [0])), shape=score.shape)
    out = filter_predictions(score, filt)
    assert out[0, 0] == 0 and out.nnz == score.nnz - 1
    assert topk_indices(out, 2)[0].tolist() == [1, 2]
    df = metrics_table(score, true, np.ones(6), K=3)
    assert list(df.index) == ["P", "nDCG", "PSP", "PSnDCG"] and list(df.columns) == ["1", "2", "3"]
