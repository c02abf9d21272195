"""Zero-compacted rows (exact_rows_mask_count / compact_write / expand) against the numpy restatement:
bit-exact mask, offsets, values and round trip, special values included."""
import numpy as np
import pytest
import torch

import oracle
from exact_b200.cpp_extension import rows as R
from helpers import normal

pytestmark = pytest.mark.gpu


def sparse_matrix(n, K, density, seed):
    rng = np.random.default_rng(seed)
    x = normal(n, K, seed)
    x[rng.random((n, K)) >= density] = 0.0
    return x


@pytest.mark.parametrize("n,K,density", [(1000, 256, 0.25), (37, 32, 0.5), (513, 64, 0.0), (200, 96, 1.0),
                                         (4099, 128, 0.03)])
def test_compact_matches_oracle_and_round_trips(n, K, density):
    x = sparse_matrix(n, K, density, 3)
    if n > 10:
        x[1, 5] = -0.0            # kept: its sign bit is set
        x[2, 0] = np.float32("nan")
        x[3, K - 1] = np.float32("inf")
        x[4, 7] = np.float32(1e-42)   # denormal
    mask, rowoff, vals = R.compact(torch.from_numpy(x).cuda())
    omask, orowoff, ovals = oracle.rows_compact(x)
    assert np.array_equal(mask.cpu().numpy().view(np.uint32), omask)
    assert np.array_equal(rowoff.cpu().numpy(), orowoff)
    nnz = int(orowoff[-1])
    assert np.array_equal(vals.cpu().numpy()[:nnz].view(np.uint32), ovals.view(np.uint32))
    out = torch.full((n, K), 7.0, device="cuda")
    R.expand(mask, rowoff, vals, n, K, n, n + 1, vals.numel(), out)
    assert np.array_equal(out.cpu().numpy().view(np.uint32), x.view(np.uint32))
    assert np.array_equal(oracle.rows_expand(omask, orowoff, ovals, K).view(np.uint32), x.view(np.uint32))


def test_expand_concatenated_shards_into_strided_rows():
    """Three shards of 40 rows (the last one short, zero padded), each with its own offsets and value
    array at a fixed stride, expanded by one launch into a matrix with a wider row pitch."""
    K, S, cap = 64, 40, 4096
    shards = [sparse_matrix(40, K, 0.3, 1), sparse_matrix(40, K, 0.2, 2), sparse_matrix(25, K, 0.4, 3)]
    mask_all = torch.zeros((3 * S, K // 32), dtype=torch.int32, device="cuda")
    rowoff_all = torch.zeros(3 * (S + 1), dtype=torch.int64, device="cuda")
    vals_all = torch.zeros(3 * cap, dtype=torch.float32, device="cuda")
    for b, xs in enumerate(shards):
        xp = np.zeros((S, K), dtype=np.float32)
        xp[:xs.shape[0]] = xs
        m, ro, v = R.compact(torch.from_numpy(xp).cuda())
        mask_all[b * S:(b + 1) * S] = m
        rowoff_all[b * (S + 1):(b + 1) * (S + 1)] = ro
        vals_all[b * cap:b * cap + v.numel()] = v
    big = torch.full((3 * S, K + 32), 9.0, device="cuda")
    R.expand(mask_all, rowoff_all, vals_all, 3 * S, K, S, S + 1, cap, big[:, :K])
    got = big.cpu().numpy()
    assert (got[:, K:] == 9.0).all()
    for b, xs in enumerate(shards):
        assert np.array_equal(got[b * S:b * S + xs.shape[0], :K], xs)
        assert (got[b * S + xs.shape[0]:(b + 1) * S, :K] == 0).all()


def test_rejects_bad_shapes():
    with pytest.raises(RuntimeError):
        R.compact(torch.zeros(8, 48, device="cuda"))
