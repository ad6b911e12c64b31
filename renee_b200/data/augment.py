"""Label-text augmentation: every label's own text becomes a training point whose positive is that label.

    python -m renee_b200.data.augment --data-dir DIR --tokenization-folder bert-base-uncased-32 --max-len 32

Creates ``<DIR>-Aug`` next to the dataset: the label files and the tokenisation folder are copied,
``trn_X_Y.txt`` gets an ``L x L`` identity appended below it, and the label tokenisations
(``lbl_*.dat``) are appended to the train token memmaps — the transformation of the reference's
``utils/CreateAugData.py`` (lines 31-107).  Copies are done in-process (the reference shells out to
``cp`` without waiting for completion) and the enlarged memmaps are written in row blocks.
"""
from __future__ import annotations

import argparse
import os
import shutil

import numpy as np
import scipy.sparse as sp

from .xcrepo import read_sparse_file, write_sparse_file


def _append_rows(dst_path: str, a_path: str, n_a: int, b_path: str, n_b: int, width: int, block: int = 1 << 18) -> None:
    a = np.memmap(a_path, dtype=np.int64, mode="r", shape=(n_a, width))
    b = np.memmap(b_path, dtype=np.int64, mode="r", shape=(n_b, width))
    tmp = dst_path + ".tmp"
    out = np.memmap(tmp, dtype=np.int64, mode="w+", shape=(n_a + n_b, width))
    for s in range(0, n_a, block):
        e = min(s + block, n_a)
        out[s:e] = a[s:e]
    for s in range(0, n_b, block):
        e = min(s + block, n_b)
        out[n_a + s: n_a + e] = b[s:e]
    out.flush()
    del out, a, b
    os.replace(tmp, dst_path)


def create_augmented_dataset(data_dir: str, tokenization_folder: str, max_len: int) -> str:
    data_dir = data_dir.rstrip("/")
    aug = data_dir + "-Aug"
    os.makedirs(aug, exist_ok=True)
    for name in ("trn_filter_labels.txt", "tst_X_Y.txt", "tst_filter_labels.txt"):
        src = os.path.join(data_dir, name)
        if os.path.exists(src):
            shutil.copyfile(src, os.path.join(aug, name))
    tok_src = os.path.join(data_dir, tokenization_folder)
    tok_dst = os.path.join(aug, tokenization_folder)
    if os.path.exists(tok_dst):
        shutil.rmtree(tok_dst)
    shutil.copytree(tok_src, tok_dst)
    trn = read_sparse_file(os.path.join(data_dir, "trn_X_Y.txt"))
    N, L = trn.shape
    aug_labels = sp.vstack((trn, sp.identity(L, dtype=np.float32, format="csr"))).tocsr()
    write_sparse_file(aug_labels, os.path.join(aug, "trn_X_Y.txt"))
    for kind in ("input_ids", "attention_mask"):
        _append_rows(os.path.join(tok_dst, f"trn_doc_{kind}.dat"), os.path.join(tok_src, f"trn_doc_{kind}.dat"), N,
                     os.path.join(tok_src, f"lbl_{kind}.dat"), L, max_len)
    return aug


def main(argv=None) -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--data-dir", type=str, required=True)
    ap.add_argument("--tokenization-folder", type=str, required=True)
    ap.add_argument("--max-len", type=int, required=True)
    a = ap.parse_args(argv)
    print("Augmented data created at:", create_augmented_dataset(a.data_dir, a.tokenization_folder, a.max_len))


if __name__ == "__main__":
    main()
