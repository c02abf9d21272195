"""Seeded synthetic inputs shared by the tests."""
import numpy as np


def relu_normal(N, D, seed):
    rng = np.random.default_rng(seed)
    return np.maximum(rng.standard_normal((N, D)).astype(np.float32), 0)


def normal(N, D, seed):
    return np.random.default_rng(seed).standard_normal((N, D)).astype(np.float32)


def uniform01(shape, seed):
    return np.random.default_rng(seed).random(shape, dtype=np.float32)


def random_csr(n_rows, n_cols, nnz, seed, with_values=True):
    rng = np.random.default_rng(seed)
    key = np.unique(rng.integers(0, n_rows * n_cols, size=nnz, dtype=np.int64))
    row, col = key // n_cols, key % n_cols
    val = rng.standard_normal(key.size).astype(np.float32) if with_values else None
    rowptr = np.zeros(n_rows + 1, np.int64)
    np.cumsum(np.bincount(row, minlength=n_rows), out=rowptr[1:])
    return rowptr, col, val


def er_graph(n, avg_deg, seed):
    """Erdos-Renyi, symmetrised, self-loops added; returns (row, col) int64 sorted by row."""
    rng = np.random.default_rng(seed)
    m = int(n * avg_deg / 2)
    a = rng.integers(0, n, size=m, dtype=np.int64)
    b = rng.integers(0, n, size=m, dtype=np.int64)
    keep = a != b
    a, b = a[keep], b[keep]
    loop = np.arange(n, dtype=np.int64)
    row = np.concatenate([a, b, loop])
    col = np.concatenate([b, a, loop])
    key = np.unique(row * n + col)
    return key // n, key % n
