"""GPU parity of the CSR SpMM (sum / mean, forward and dense-operand gradient) against the oracle."""
import numpy as np
import pytest
import torch

import oracle
from exact_b200 import SparseTensor, config, qmatmul
from exact_b200.cpp_extension import spmm as S
from helpers import normal, random_csr

pytestmark = pytest.mark.gpu


def t(a, dtype=None):
    x = torch.from_numpy(np.ascontiguousarray(a)).cuda()
    return x if dtype is None else x.to(dtype)


@pytest.mark.parametrize("idx", [torch.int64, torch.int32])
@pytest.mark.parametrize("reduce", ["sum", "mean"])
@pytest.mark.parametrize("with_values", [True, False])
@pytest.mark.parametrize("K", [128, 602, 256, 100, 40, 16, 13, 1])
def test_forward_bit_exact(K, with_values, reduce, idx):
    # test/test_op.py:506-562 shapes: 10,000 nodes, 50,000 edges
    rowptr, col, val = random_csr(10000, 10000, 50000, 3, with_values)
    mat = normal(10000, K, 4)
    fn = S.spmm_sum_fw if reduce == "sum" else S.spmm_mean_fw
    args = (None, t(rowptr, idx), t(col, idx), None if val is None else t(val))
    out = fn(*args, None, None, t(mat)) if reduce == "sum" else fn(*args, None, None, None, t(mat))
    ref = oracle.spmm(rowptr, col, val, mat, reduce)
    # same per-row summation order and one FMA per edge as the oracle: bit-exact
    assert np.array_equal(out.cpu().numpy(), ref)


@pytest.mark.parametrize("with_values", [True, False])
@pytest.mark.parametrize("K", [256, 100, 602])
def test_hub_rows_and_empty_rows(K, with_values):
    """A 2,500-edge hub row (cut into pieces summed by separate warps), ordinary rows and empty rows.
    Rows up to the threshold keep the reference's summation order (bit-exact); the hub rows are a
    regrouped fp32 sum (1e-5 of the row's largest entry)."""
    n = 3000
    rng = np.random.default_rng(9)
    hub = np.stack([np.zeros(2500, np.int64), rng.choice(n, 2500, replace=False)])
    hub2 = np.stack([np.full(700, 2999, np.int64), rng.choice(n, 700, replace=False)])
    rest = rng.integers(0, n, (2, 6000))
    rest = rest[:, (rest[0] > 100) & (rest[0] < 2999)]        # rows 1..100 empty
    e = np.concatenate([hub, hub2, rest], 1)
    key = np.unique(e[0] * n + e[1])
    row, col = key // n, key % n
    rowptr = np.zeros(n + 1, np.int64)
    np.cumsum(np.bincount(row, minlength=n), out=rowptr[1:])
    val = rng.standard_normal(col.size).astype(np.float32) if with_values else None
    mat = normal(n, K, 10)
    long = np.diff(rowptr) > 512
    assert long.sum() == 2
    for reduce in ("sum", "mean"):
        ref = oracle.spmm(rowptr, col, val, mat, reduce)
        for thr in (512, 0):
            config.spmm_long_row = thr
            out = S._spmm(t(rowptr), t(col), None if val is None else t(val), t(mat), reduce).cpu().numpy()
            if thr == 0:
                assert np.array_equal(out, ref)
            else:
                assert np.array_equal(out[~long], ref[~long])
                # a regrouped fp32 sum of ~10^3 terms: error relative to the size of the row, not of
                # each (possibly cancelling) element
                err = np.abs(out[long] - ref[long]).max(1)
                assert np.all(err <= 1e-5 * np.abs(ref[long]).max(1))
    config.spmm_long_row = 256


@pytest.mark.parametrize("reduce", ["sum", "mean"])
@pytest.mark.parametrize("with_values", [True, False])
def test_qmatmul_forward_and_grad(reduce, with_values):
    config.compress_activation = True
    config.kept_frac = 1.0
    n, K = 5000, 128
    rowptr, col, val = random_csr(n, n, 40000, 5, with_values)
    row = np.repeat(np.arange(n), np.diff(rowptr))
    adj = SparseTensor(row=t(row), col=t(col), value=None if val is None else t(val), sparse_sizes=(n, n),
                       is_sorted=True)
    mat = normal(n, K, 6)
    g = normal(n, K, 7)
    x = t(mat).requires_grad_()
    out = qmatmul(adj, x, reduce)
    out.backward(t(g))
    assert np.array_equal(out.detach().cpu().numpy(), oracle.spmm(rowptr, col, val, mat, reduce))
    ref_g = oracle.spmm_bw_mat(rowptr, col, val, g, n, reduce)
    np.testing.assert_allclose(x.grad.cpu().numpy(), ref_g, rtol=1e-6, atol=1e-6)
    # and against torch's own sparse product
    A = torch.sparse_csr_tensor(t(rowptr), t(col), t(val) if with_values else torch.ones(col.size, device="cuda"),
                                size=(n, n))
    dense = A.to_dense()
    if reduce == "mean":
        dense = dense / torch.from_numpy(np.maximum(np.diff(rowptr), 1)).cuda().float()[:, None]
    torch.testing.assert_close(out.detach(), dense @ t(mat), rtol=1e-4, atol=1e-4)
    torch.testing.assert_close(x.grad, dense.t() @ t(g), rtol=1e-4, atol=1e-4)


@pytest.mark.parametrize("reduce", ["sum", "mean"])
@pytest.mark.parametrize("with_values", [True, False])
@pytest.mark.parametrize("K", [48, 64, 40, 32, 24, 16, 8, 4])
def test_regrouped_sum_for_narrow_operands(K, with_values, reduce):
    """EXACT_SPMM_REGROUP: operands of at most 64 / 32 / 16 columns gather two / four / eight edges per load
    instruction and add the interleaved partial sums; the result equals the edge-order sum up to fp32
    reassociation, hub rows (cut into pieces) and empty rows included.  Wider operands ignore the flag and
    stay bit-exact."""
    n = 4000
    rng = np.random.default_rng(11)
    hub = np.stack([np.zeros(1500, np.int64), rng.choice(n, 1500, replace=False)])
    rest = rng.integers(0, n, (2, 30000))
    rest = rest[:, rest[0] > 50]                                # rows 1..50 empty
    e = np.concatenate([hub, rest], 1)
    key = np.unique(e[0] * n + e[1])
    row, col = key // n, key % n
    rowptr = np.zeros(n + 1, np.int64)
    np.cumsum(np.bincount(row, minlength=n), out=rowptr[1:])
    val = rng.standard_normal(col.size).astype(np.float32) if with_values else None
    mat = normal(n, K, 12)
    ref = oracle.spmm(rowptr, col, val, mat, reduce)
    out = S._spmm(t(rowptr), t(col), None if val is None else t(val), t(mat), reduce, regroup=True).cpu().numpy()
    absval = np.ones(col.size, np.float32) if val is None else np.abs(val)
    scale = oracle.spmm(rowptr, col, absval, np.abs(mat), reduce) + 1e-30
    assert np.all(np.abs(out - ref) <= 2e-6 * scale)
    assert np.array_equal(out[1:51], np.zeros((50, K), np.float32))
    wide = normal(n, 128, 13)
    strict = S._spmm(t(rowptr), t(col), None if val is None else t(val), t(wide), reduce).cpu().numpy()
    flagged = S._spmm(t(rowptr), t(col), None if val is None else t(val), t(wide), reduce, regroup=True).cpu().numpy()
    assert np.array_equal(strict, flagged)


@pytest.mark.parametrize("reduce", ["sum", "mean"])
@pytest.mark.parametrize("K,regroup", [(32, True), (8, True), (64, True), (128, False), (100, False), (13, False)])
def test_routed_output_equals_local_result_then_scatter(K, regroup, reduce):
    """exact_spmm_split_routed: every result row goes straight into columns col0 .. of row r % shard of the buffer
    of its owner r // shard (here three local buffers standing for three ranks).  Same bits as the local result
    cut into row blocks; hub rows (pieces + ordered sum) and empty rows included; the other columns of the
    buffers stay untouched."""
    n, shard, col0, ldd = 4000, 1336, 4 * ((K + 3) // 4), 3 * 4 * ((K + 3) // 4) + 8
    rng = np.random.default_rng(31)
    hub = np.stack([np.full(1500, 1400, np.int64), rng.choice(n, 1500, replace=False)])
    rest = rng.integers(0, n, (2, 30000))
    rest = rest[:, rest[0] > 50]
    e = np.concatenate([hub, rest], 1)
    key = np.unique(e[0] * n + e[1])
    row, col = key // n, key % n
    rowptr = np.zeros(n + 1, np.int64)
    np.cumsum(np.bincount(row, minlength=n), out=rowptr[1:])
    mat = t(normal(n, K, 32))
    local = S._spmm(t(rowptr), t(col), None, mat, reduce, regroup=regroup)
    bufs = [torch.full((shard, ldd), -7.0, device="cuda") for _ in range(3)]
    assert S._spmm(t(rowptr), t(col), None, mat, reduce, regroup=regroup,
                   route=(shard, col0, ldd, [b.data_ptr() for b in bufs])) is None
    for q, b in enumerate(bufs):
        rows = local[q * shard:(q + 1) * shard]
        assert torch.equal(b[:rows.size(0), col0:col0 + K], rows)
        assert bool((b[:, :col0] == -7.0).all()) and bool((b[:, col0 + K:] == -7.0).all())
        assert bool((b[rows.size(0):] == -7.0).all())


@pytest.mark.parametrize("K", [256, 64])
def test_power_law_graph_with_many_out_of_order_pieces(K):
    """An R-MAT graph of the benchmark's skew: 120,000 nodes, ~6 M edges, hub rows of 10^4 edges cut into dozens
    of pieces that are listed (= processed) by the column of their first edge, not in row order (item_slot).
    Rows up to the threshold are bit-exact against the oracle; hub rows are a regrouped fp32 sum."""
    from exact_b200 import graphs
    adj = graphs.rmat(120_000, 3_000_000, 5, "cuda", self_loops=False)
    adj.to_int32_()
    rowptr, col, _ = adj.csr()
    plan = S.long_row_plan(rowptr, 256, col)
    assert plan is not None and plan["n_items"] > 1000
    pieces = (plan["long_item_ptr"][1:] - plan["long_item_ptr"][:-1])
    assert int(pieces.max()) >= 10
    slot = plan["item_slot"].cpu().numpy()
    assert not np.array_equal(slot, np.arange(slot.size)) and np.array_equal(np.sort(slot), np.arange(slot.size))
    mat = normal(120_000, K, 21)
    rp, cl = rowptr.cpu().numpy().astype(np.int64), col.cpu().numpy().astype(np.int64)
    long = np.diff(rp) > 256
    for reduce in ("mean", "sum"):
        out = S._spmm(rowptr, col, None, t(mat), reduce).cpu().numpy()
        ref = oracle.spmm(rp, cl, None, mat, reduce)
        assert np.array_equal(out[~long], ref[~long])
        err = np.abs(out[long] - ref[long]).max(1)
        assert np.all(err <= 1e-5 * np.abs(ref[long]).max(1) + 1e-6 * np.sqrt(np.diff(rp)[long]) * (reduce == "sum"))


@pytest.mark.parametrize("idx", [torch.int64, torch.int32])
@pytest.mark.parametrize("reduce", ["sum", "mean"])
@pytest.mark.parametrize("K", [128, 100, 40, 13])
def test_value_gradient_bit_exact(K, reduce, idx):
    """spmm_value_bw (spmm_cuda.cu:172-209): the same lane-strided FMAs and shuffle tree as the reference."""
    rowptr, col, val = random_csr(5000, 5000, 40000, 3, True)
    row = np.repeat(np.arange(5000), np.diff(rowptr))
    mat, g = normal(5000, K, 4), normal(5000, K, 5)
    out = S.spmm_value_bw(t(row, idx), t(rowptr, idx), t(col, idx), t(mat), t(g), reduce)
    assert np.array_equal(out.cpu().numpy(), oracle.spmm_value_bw(rowptr, col, mat, g, reduce))


@pytest.mark.parametrize("reduce", ["sum", "mean"])
def test_qmatmul_edge_value_gradient(reduce):
    """Edge values that require grad: the saved dense operand is dequantised (and projected back) and the value
    gradient computed from it (ops.py:291-307, 341-371); with compression off it is exact."""
    config.compress_activation = False
    n, K = 3000, 64
    rowptr, col, val = random_csr(n, n, 20000, 5, True)
    row = np.repeat(np.arange(n), np.diff(rowptr))
    v = t(val).requires_grad_()
    adj = SparseTensor(row=t(row), col=t(col), value=v, sparse_sizes=(n, n), is_sorted=True)
    mat, g = normal(n, K, 6), normal(n, K, 7)
    x = t(mat).requires_grad_()
    out = qmatmul(adj, x, reduce)
    out.backward(t(g))
    assert np.array_equal(v.grad.cpu().numpy(), oracle.spmm_value_bw(rowptr, col, mat, g, reduce))
    config.compress_activation = True


@pytest.mark.parametrize("idx", [torch.int64, torch.int32])
@pytest.mark.parametrize("reduce", ["max", "min"])
@pytest.mark.parametrize("with_values", [True, False])
@pytest.mark.parametrize("K", [128, 40, 13])
def test_max_min_forward_and_grad(K, with_values, reduce, idx):
    """spmm_max / spmm_min (test/test_op.py:506-562 asserts them against torch_sparse): values and the position
    of the winning edge equal the oracle's (the first edge of a tie wins, empty rows give 0 and arg = nnz);
    the gradient goes to the winning source rows (spmm.cc:159-193)."""
    n = 3000
    rowptr, col, val = random_csr(n, n, 15000, 3, with_values)     # average degree 5: some rows are empty
    mat = normal(n, K, 4)
    mat[:, 0] = 1.0                                                # ties in column 0
    fn = S.spmm_max_fw if reduce == "max" else S.spmm_min_fw
    out, arg = fn(t(rowptr, idx), t(col, idx), None if val is None else t(val), t(mat))
    ref_out, ref_arg = oracle.spmm_minmax(rowptr, col, val, mat, reduce)
    assert np.array_equal(out.cpu().numpy(), ref_out)
    assert np.array_equal(arg.cpu().numpy().astype(np.int64), ref_arg)
    # autograd through qmatmul with compression off: d out / d mat scatters g to the winners
    config.compress_activation = False
    row = np.repeat(np.arange(n), np.diff(rowptr))
    adj = SparseTensor(row=t(row), col=t(col), value=None if val is None else t(val), sparse_sizes=(n, n), is_sorted=True)
    x = t(mat).requires_grad_()
    g = normal(n, K, 5)
    qmatmul(adj, x, reduce).backward(t(g))
    ref_g = np.zeros((n, K), np.float64)
    valid = ref_arg < col.size
    w = np.ones(col.size, np.float32) if val is None else val
    rr, cc = np.nonzero(valid)
    np.add.at(ref_g, (col[ref_arg[rr, cc]], cc), (w[ref_arg[rr, cc]] * g[rr, cc]).astype(np.float64))
    np.testing.assert_allclose(x.grad.cpu().numpy(), ref_g, rtol=1e-5, atol=1e-5)
    config.compress_activation = True
