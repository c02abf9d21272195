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


@pytest.mark.parametrize("n,K,P", [(1000, 256, 8), (999, 100, 8), (512, 48, 4), (300, 256, 2), (77, 100, 2)])
def test_feature_parallel_exchange_kernels(n, K, P):
    """exact_cols_scatter / exact_rows_scatter with all P "ranks" played on one device: column slices of every
    shard's rows to every rank, then row blocks of every rank's slice back, reproduce the matrix (padding zero)."""
    x = normal(n, K, 5)
    shard = ((n + P - 1) // P + 7) // 8 * 8
    Kp = ((K + P - 1) // P + 3) // 4 * 4
    scale = (np.random.default_rng(6).random(n).astype(np.float32) + 0.5)
    inb = [torch.full((P * shard, Kp), 7.0, device="cuda") for _ in range(P)]
    outb = [torch.full((shard, P * Kp), 9.0, device="cuda") for _ in range(P)]
    xt, st = t(x), t(scale)
    for r in range(P):                      # rank r scatters its rows' column slices to everyone
        r0, r1 = min(r * shard, n), min(r * shard + shard, n)
        if r1 > r0:
            R.cols_scatter(xt[r0:r1], st[r0:r1], r0, Kp, [b.data_ptr() for b in inb])
    xs = (x * scale[:, None]).astype(np.float32)
    padded = np.zeros((n, P * Kp), np.float32)
    padded[:, :K] = xs
    for q in range(P):
        assert np.array_equal(inb[q][:n].cpu().numpy(), padded[:, q * Kp:(q + 1) * Kp])
        assert float(inb[q][n:].min()) == 7.0 if n < P * shard else True
    for q in range(P):                      # rank q sends the row blocks of its slice back to their owners
        R.rows_scatter(inb[q][:n].contiguous(), shard, q * Kp, P * Kp, [b.data_ptr() for b in outb])
    for r in range(P):
        r0, r1 = min(r * shard, n), min(r * shard + shard, n)
        assert np.array_equal(outb[r][:r1 - r0].cpu().numpy(), padded[r0:r1])
