"""Compact rows (exact_crows_pack / exact_crows_unpack) against the numpy restatement, and the SpMM that gathers
them (exact_spmm_crows) against the dense SpMM and the oracle: bit-exact, special values included."""
import numpy as np
import pytest
import torch

import oracle
from exact_b200 import config
from exact_b200.cpp_extension import rows as R
from exact_b200.cpp_extension import spmm as S
from helpers import normal, random_csr

pytestmark = pytest.mark.gpu


def sparse_matrix(n, K, density, seed):
    rng = np.random.default_rng(seed)
    x = normal(n, K, seed)
    x[rng.random((n, K)) >= density] = 0.0
    return x


def t(a, dtype=None):
    x = torch.from_numpy(np.ascontiguousarray(a)).cuda()
    return x if dtype is None else x.to(dtype)


@pytest.mark.parametrize("n,K,density", [(1000, 256, 0.25), (37, 32, 0.5), (513, 64, 0.0), (200, 96, 1.0),
                                         (4099, 128, 0.03), (300, 100, 0.3), (65, 8, 0.5), (1, 256, 1.0)])
@pytest.mark.parametrize("scaled", [False, True])
def test_pack_matches_oracle_and_round_trips(n, K, density, scaled):
    x = sparse_matrix(n, K, density, 3)
    if n > 10:
        x[1, 5] = -0.0            # kept: its sign bit is set
        x[2, 0] = np.float32("nan")
        x[3, K - 1] = np.float32("inf")
        x[4, 7] = np.float32(1e-42)   # denormal
    scale = (np.random.default_rng(5).random(n).astype(np.float32) + 0.5) if scaled else None
    kept = torch.zeros(1, dtype=torch.int64, device="cuda")
    cr = R.crows_pack(t(x), None if scale is None else t(scale), kept_total=kept)
    ref = oracle.crows_pack(x, scale)
    got = cr.buf.cpu().numpy().reshape(n, -1)
    used = oracle.crows_used_mask(ref, K)
    assert got.shape == ref.shape
    assert np.array_equal(got[used], ref[used])
    xs = x if scale is None else (x * scale[:, None]).astype(np.float32)
    assert int(kept.item()) == int((xs.view(np.uint32) != 0).sum())
    dense = R.crows_unpack(cr).cpu().numpy()
    assert np.array_equal(dense.view(np.uint32), xs.view(np.uint32))


def test_pack_into_offset_slots_and_two_destinations():
    """Two shards written into two buffers at their global slot indices (what row shards do with each other's
    memory) reproduce the pack of the whole matrix."""
    n, K = 96, 128
    x = sparse_matrix(n, K, 0.25, 9)
    a, b = R.crows_alloc(n, K, "cuda"), R.crows_alloc(n, K, "cuda")
    a.buf.zero_(), b.buf.zero_()
    for r0, r1 in ((0, 40), (40, 96)):
        R.crows_pack(t(x[r0:r1]), row0=r0, dst_ptrs=[a.ptr(), b.ptr()])
    whole = R.crows_pack(t(x))
    used = oracle.crows_used_mask(oracle.crows_pack(x), K)
    for buf in (a, b):
        assert np.array_equal(buf.buf.cpu().numpy().reshape(n, -1)[used], whole.buf.cpu().numpy().reshape(n, -1)[used])


@pytest.mark.parametrize("idx", [torch.int64, torch.int32])
@pytest.mark.parametrize("reduce", ["sum", "mean"])
@pytest.mark.parametrize("with_values", [True, False])
@pytest.mark.parametrize("K,density", [(256, 0.25), (128, 0.6), (64, 1.0), (100, 0.25), (256, 0.0), (8, 0.5), (36, 0.9)])
def test_spmm_over_compact_rows_is_bit_exact(K, density, with_values, reduce, idx):
    rowptr, col, val = random_csr(10000, 10000, 50000, 3, with_values)
    mat = sparse_matrix(10000, K, density, 4)
    mat[7, 3] = -0.0
    cr = R.crows_pack(t(mat))
    args = (t(rowptr, idx), t(col, idx), None if val is None else t(val))
    out = S._spmm(*args, cr, reduce).cpu().numpy()
    dense = S._spmm(*args, t(mat), reduce).cpu().numpy()
    ref = oracle.spmm(rowptr, col, val, mat, reduce)
    assert np.array_equal(out.view(np.uint32), dense.view(np.uint32))
    assert np.array_equal(out, ref)


@pytest.mark.parametrize("with_values", [True, False])
def test_spmm_over_compact_rows_with_hub_rows(with_values):
    """Long rows are cut into the same pieces as in the dense kernel, so the two agree bit for bit there too."""
    n, K = 3000, 256
    rng = np.random.default_rng(9)
    hub = np.stack([np.zeros(2500, np.int64), rng.choice(n, 2500, replace=False)])
    hub2 = np.stack([np.full(700, 2999, np.int64), rng.choice(n, 700, replace=False)])
    rest = rng.integers(0, n, (2, 6000))
    rest = rest[:, (rest[0] > 100) & (rest[0] < 2999)]
    e = np.concatenate([hub, hub2, rest], 1)
    key = np.unique(e[0] * n + e[1])
    row, col = key // n, key % n
    rowptr = np.zeros(n + 1, np.int64)
    np.cumsum(np.bincount(row, minlength=n), out=rowptr[1:])
    val = rng.standard_normal(col.size).astype(np.float32) if with_values else None
    mat = sparse_matrix(n, K, 0.25, 10)
    cr = R.crows_pack(t(mat))
    for reduce in ("sum", "mean"):
        for thr in (512, 0):
            config.spmm_long_row = thr
            args = (t(rowptr), t(col), None if val is None else t(val))
            out = S._spmm(*args, cr, reduce).cpu().numpy()
            dense = S._spmm(*args, t(mat), reduce).cpu().numpy()
            assert np.array_equal(out.view(np.uint32), dense.view(np.uint32))
    config.spmm_long_row = 256
