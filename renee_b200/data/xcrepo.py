"""Readers/writers for the Extreme Classification Repository on-disk formats the reference uses.

* sparse label files ``trn_X_Y.txt`` / ``tst_X_Y.txt``: first line ``"<rows> <cols>"``, then one
  line per row of space-separated ``col:val`` pairs (read through pyxclib's ``read_sparse_file`` at
  reference main.py:50-51);
* ``tst_filter_labels.txt``: whitespace-separated ``row col`` integer pairs (main.py:62-64);
* token files ``{trn_doc,tst_doc,lbl}_{input_ids,attention_mask}.dat``: raw little-endian int64
  arrays ``[num_points, maxlen]`` in a folder ``{tokenizer_type}-{maxlen}`` (dl_base.py:886-889,
  utils/CreateTokenizedFiles.py:63-69).
"""
from __future__ import annotations

import os

import numpy as np
import scipy.sparse as sp


def read_sparse_file(path: str, dtype=np.float32) -> sp.csr_matrix:
    with open(path, "r") as f:
        header = f.readline().split()
        rows, cols = int(header[0]), int(header[1])
        indptr = np.zeros(rows + 1, dtype=np.int64)
        idx_chunks, val_chunks = [], []
        r = 0
        for line in f:
            if r >= rows:
                break
            toks = line.split()
            if toks:
                pairs = [t.split(":") for t in toks]
                idx_chunks.append(np.fromiter((int(p[0]) for p in pairs), dtype=np.int64, count=len(pairs)))
                val_chunks.append(np.fromiter((float(p[1]) if len(p) > 1 else 1.0 for p in pairs),
                                              dtype=dtype, count=len(pairs)))
            indptr[r + 1] = indptr[r] + len(toks)
            r += 1
        indptr[r + 1:] = indptr[r]
    indices = np.concatenate(idx_chunks) if idx_chunks else np.zeros(0, dtype=np.int64)
    data = np.concatenate(val_chunks) if val_chunks else np.zeros(0, dtype=dtype)
    return sp.csr_matrix((data, indices, indptr), shape=(rows, cols))


def write_sparse_file(mat: sp.spmatrix, path: str) -> None:
    mat = sp.csr_matrix(mat)
    with open(path, "w") as f:
        f.write(f"{mat.shape[0]} {mat.shape[1]}\n")
        for r in range(mat.shape[0]):
            lo, hi = mat.indptr[r], mat.indptr[r + 1]
            f.write(" ".join(f"{c}:{v:.5f}" for c, v in zip(mat.indices[lo:hi], mat.data[lo:hi])))
            f.write("\n")


def read_filter_file(path: str, shape: tuple[int, int]) -> sp.csr_matrix:
    """``(row, col)`` pairs → CSR of ones.  A missing or empty file yields an empty matrix."""
    if not os.path.exists(path) or os.path.getsize(path) == 0:
        return sp.csr_matrix(shape, dtype=np.float32)
    flat = np.fromfile(path, sep=" ").astype(np.int64)
    pairs = flat.reshape(-1, 2).T
    return sp.coo_matrix((np.ones(pairs.shape[1], dtype=np.float32), (pairs[0], pairs[1])), shape).tocsr()


def write_filter_file(pairs: np.ndarray, path: str) -> None:
    pairs = np.asarray(pairs, dtype=np.int64).reshape(-1, 2)
    with open(path, "w") as f:
        for r, c in pairs:
            f.write(f"{r} {c}\n")


def tokenizer_folder(tf_name: str) -> str:
    """Tokenisation-folder prefix derived from the encoder name (reference main.py:67-74)."""
    if "roberta" in tf_name:
        return "roberta-base"
    if "bert" in tf_name:
        return "bert-base-uncased"
    if "MiniLM" in tf_name:
        return "miniLM_L6"
    return tf_name


def write_token_files(folder: str, prefix: str, input_ids: np.ndarray, attention_mask: np.ndarray) -> None:
    os.makedirs(folder, exist_ok=True)
    np.ascontiguousarray(input_ids, dtype=np.int64).tofile(os.path.join(folder, f"{prefix}_input_ids.dat"))
    np.ascontiguousarray(attention_mask, dtype=np.int64).tofile(os.path.join(folder, f"{prefix}_attention_mask.dat"))


class PreTokDataset:
    """Pre-tokenised text held in int64 memmaps, opened lazily on first access so that forked
    loader workers do not duplicate the mapping (reference dl_base.py:864-896)."""

    def __init__(self, folder: str, labels: sp.csr_matrix | None, num_points: int, maxlen: int, doc_type: str = "trn"):
        self.folder = folder
        self.labels = labels
        self.num_points = int(num_points)
        self.maxlen = int(maxlen)
        self.doc_type = doc_type
        self._ids = None
        self._mask = None

    def __len__(self) -> int:
        return self.num_points

    def __getitem__(self, index: int) -> int:
        return index

    def _open(self):
        if self._ids is None:
            shape = (self.num_points, self.maxlen)
            self._ids = np.memmap(os.path.join(self.folder, f"{self.doc_type}_doc_input_ids.dat"),
                                  mode="r", shape=shape, dtype=np.int64)
            self._mask = np.memmap(os.path.join(self.folder, f"{self.doc_type}_doc_attention_mask.dat"),
                                   mode="r", shape=shape, dtype=np.int64)

    def get_fts(self, indices) -> tuple[np.ndarray, np.ndarray]:
        self._open()
        indices = np.asarray(indices, dtype=np.int64)
        return np.asarray(self._ids[indices]), np.asarray(self._mask[indices])


class InMemoryDataset:
    """Same interface as :class:`PreTokDataset` over arrays already in memory (synthetic runs)."""

    def __init__(self, input_ids: np.ndarray, attention_mask: np.ndarray, labels: sp.csr_matrix | None):
        self.input_ids = input_ids
        self.attention_mask = attention_mask
        self.labels = labels
        self.num_points = int(input_ids.shape[0])
        self.maxlen = int(input_ids.shape[1])

    def __len__(self) -> int:
        return self.num_points

    def __getitem__(self, index: int) -> int:
        return index

    def get_fts(self, indices) -> tuple[np.ndarray, np.ndarray]:
        indices = np.asarray(indices, dtype=np.int64)
        return self.input_ids[indices], self.attention_mask[indices]


def write_synthetic_dataset(data_dir: str, tf_name: str, maxlen: int, trn, tst, filter_pairs=None) -> None:
    """Write ``(input_ids, mask, labels)`` triples for train and test in the repository layout."""
    os.makedirs(data_dir, exist_ok=True)
    folder = os.path.join(data_dir, f"{tokenizer_folder(tf_name)}-{maxlen}")
    write_token_files(folder, "trn_doc", trn[0], trn[1])
    write_token_files(folder, "tst_doc", tst[0], tst[1])
    write_sparse_file(trn[2], os.path.join(data_dir, "trn_X_Y.txt"))
    write_sparse_file(tst[2], os.path.join(data_dir, "tst_X_Y.txt"))
    write_filter_file(np.zeros((0, 2), dtype=np.int64) if filter_pairs is None else filter_pairs,
                      os.path.join(data_dir, "tst_filter_labels.txt"))
