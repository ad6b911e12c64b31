import numpy as np
import scipy.sparse as sp


def read_sparse_file(path, dtype=np.float32):
    with open(path) as f:
        rows, cols = map(int, f.readline().split())
        indptr, idx, val = [0], [], []
        for line in f:
            for tok in line.split():
                c, v = tok.split(":")
                idx.append(int(c)); val.append(float(v))
            indptr.append(len(idx))
    while len(indptr) < rows + 1:
        indptr.append(len(idx))
    return sp.csr_matrix((np.array(val, dtype=dtype), np.array(idx, dtype=np.int64), np.array(indptr[: rows + 1])),
                         shape=(rows, cols))
