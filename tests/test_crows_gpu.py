"""Compact rows (exact_crows_pack / exact_crows_unpack), the form in which row shards write their mostly-zero
operands into each other's memory, against the numpy restatement: bit-exact, special values included."""
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
        if not scaled:            # a scaled NaN is the GPU's canonical NaN, not numpy's: same value, other bits
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


def test_unpack_into_a_larger_buffer_overwrites_stale_rows():
    n, K = 500, 256
    x = sparse_matrix(n, K, 0.25, 11)
    cr = R.crows_pack(t(x))
    out = torch.full((n + 12, K), 7.0, device="cuda")
    got = R.crows_unpack(cr, n, out=out)
    assert got.data_ptr() == out.data_ptr() and np.array_equal(got.cpu().numpy(), x)
    assert float(out[n:].min()) == 7.0
