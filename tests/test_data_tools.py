"""Tokenisation and label-text augmentation tools (reference utils/CreateTokenizedFiles.py, CreateAugData.py)."""
import os

import numpy as np
import scipy.sparse as sp

from renee_b200.data import xcrepo
from renee_b200.data.augment import create_augmented_dataset
from renee_b200.data.tokenize_files import tokenize_to_memmap


def _fake_encode(texts, max_len):
    ids = np.zeros((len(texts), max_len), dtype=np.int64)
    mask = np.zeros_like(ids)
    for r, t in enumerate(texts):
        toks = [101] + [1000 + (hash(w) % 500) for w in t.split()][: max_len - 2] + [102]
        ids[r, : len(toks)] = toks
        mask[r, : len(toks)] = 1
    return ids, mask


def test_tokenize_to_memmap_layout(tmp_path):
    texts = [f"title number {i} with some words" for i in range(57)]
    folder = str(tmp_path / "bert-base-uncased-8")
    n, w = tokenize_to_memmap(texts, folder, "trn_doc", 8, "", chunk=10, encode_fn=_fake_encode)
    assert (n, w) == (57, 8)
    ids = np.fromfile(os.path.join(folder, "trn_doc_input_ids.dat"), dtype=np.int64).reshape(57, 8)
    am = np.fromfile(os.path.join(folder, "trn_doc_attention_mask.dat"), dtype=np.int64).reshape(57, 8)
    assert (ids[:, 0] == 101).all() and ((ids != 0) == (am == 1)).all() and am.sum(1).max() <= 8
    ds = xcrepo.PreTokDataset(folder, None, 57, 8, "trn")
    assert (ds.get_fts([5])[0][0] == ids[5]).all()


def test_augmentation_appends_identity_and_label_tokens(tmp_path):
    d = str(tmp_path / "LF-Toy-8")
    N, L, W = 6, 4, 8
    labels = sp.random(N, L, density=0.4, format="csr", random_state=0, dtype=np.float32)
    labels.data[:] = 1
    tok = os.path.join(d, "bert-base-uncased-8")
    xcrepo.write_token_files(tok, "trn_doc", np.arange(N * W).reshape(N, W), np.ones((N, W), dtype=np.int64))
    xcrepo.write_token_files(tok, "tst_doc", np.arange(2 * W).reshape(2, W), np.ones((2, W), dtype=np.int64))
    xcrepo.write_token_files(tok, "lbl", 900 + np.arange(L * W).reshape(L, W), np.ones((L, W), dtype=np.int64))
    xcrepo.write_sparse_file(labels, os.path.join(d, "trn_X_Y.txt"))
    xcrepo.write_sparse_file(labels[:2], os.path.join(d, "tst_X_Y.txt"))
    xcrepo.write_filter_file(np.array([[0, 1]]), os.path.join(d, "tst_filter_labels.txt"))
    aug = create_augmented_dataset(d, "bert-base-uncased-8", W)
    assert aug.endswith("LF-Toy-8-Aug")
    y = xcrepo.read_sparse_file(os.path.join(aug, "trn_X_Y.txt"))
    assert y.shape == (N + L, L) and (y[:N] != labels).nnz == 0
    assert (y[N:].toarray() == np.eye(L)).all()
    ids = np.fromfile(os.path.join(aug, "bert-base-uncased-8", "trn_doc_input_ids.dat"), dtype=np.int64).reshape(N + L, W)
    assert (ids[:N] == np.arange(N * W).reshape(N, W)).all() and (ids[N:] == 900 + np.arange(L * W).reshape(L, W)).all()
    assert os.path.exists(os.path.join(aug, "tst_filter_labels.txt"))
    # the original dataset is untouched
    assert os.path.getsize(os.path.join(tok, "trn_doc_input_ids.dat")) == N * W * 8
