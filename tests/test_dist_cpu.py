"""Host logic of the row-partitioned multi-GPU path, exercised with two gloo ranks on CPU.  The SpMM
kernel call is replaced by the CPU oracle (the test checks the sharding, the all-gathers, the transposed
slices and the gradient all-reduce, not the kernel)."""
import os
import socket

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from helpers import normal, random_csr


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _oracle_spmm(rowptr, col, value, mat, reduce):
    import oracle
    out = oracle.spmm(rowptr.numpy().astype(np.int64), col.numpy().astype(np.int64),
                      None if value is None else value.numpy(), mat.detach().numpy(), reduce)
    return torch.from_numpy(out)


def _worker(rank, world, port, reduce, with_values, n, K, result_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import exact_b200
    from exact_b200 import SparseTensor, config, qmatmul
    from exact_b200 import dist as xdist
    from exact_b200.cpp_extension import spmm as ext_spmm
    ext_spmm._spmm = _oracle_spmm          # CPU stand-in for the CUDA kernel
    xdist.ext_spmm._spmm = _oracle_spmm

    rowptr, col, val = random_csr(n, n, 6 * n, 3, with_values)
    row = np.repeat(np.arange(n), np.diff(rowptr))
    full = SparseTensor(row=torch.from_numpy(row), col=torch.from_numpy(col),
                        value=None if val is None else torch.from_numpy(val), sparse_sizes=(n, n), is_sorted=True)
    adj = xdist.shard_graph(full, reduce, rank, world)
    assert adj.row_start % 8 == 0 and config.row_offset == adj.row_start
    x_full = torch.from_numpy(normal(n, K, 4))
    g_full = torch.from_numpy(normal(n, K, 5))
    x = x_full[adj.row_start:adj.row_end].clone().requires_grad_()
    out = qmatmul(adj, x, reduce)
    out.backward(g_full[adj.row_start:adj.row_end])
    # a replicated parameter whose gradient is summed over ranks
    w = torch.nn.Parameter(torch.ones(3))
    w.grad = torch.full((3,), float(rank + 1))
    xdist.allreduce_gradients([w])
    torch.save({"out": out.detach(), "gx": x.grad, "r0": adj.row_start, "r1": adj.row_end, "wgrad": w.grad},
               os.path.join(result_dir, f"rank{rank}.pt"))
    dist.barrier()
    dist.destroy_process_group()


def _run(reduce, with_values, tmp_path, n=203, K=16, world=2):
    import oracle
    port = _free_port()
    mp.spawn(_worker, args=(world, port, reduce, with_values, n, K, str(tmp_path)), nprocs=world, join=True)
    parts = [torch.load(os.path.join(tmp_path, f"rank{r}.pt")) for r in range(world)]
    rowptr, col, val = random_csr(n, n, 6 * n, 3, with_values)
    x, g = normal(n, K, 4), normal(n, K, 5)
    ref_out = oracle.spmm(rowptr, col, val, x, reduce)
    ref_gx = oracle.spmm_bw_mat(rowptr, col, val, g, n, reduce)
    out = torch.cat([p["out"] for p in parts]).numpy()
    gx = torch.cat([p["gx"] for p in parts]).numpy()
    assert parts[0]["r0"] == 0 and parts[0]["r1"] == parts[1]["r0"] and parts[-1]["r1"] == n
    assert np.array_equal(out, ref_out)              # same per-row order on every shard
    np.testing.assert_allclose(gx, ref_gx, rtol=1e-6, atol=1e-6)
    for p in parts:
        assert torch.equal(p["wgrad"], torch.full((3,), 3.0))


def test_sharded_mean_no_values(tmp_path):
    _run("mean", False, tmp_path)


def test_sharded_sum_with_values(tmp_path):
    _run("sum", True, tmp_path)


def test_shard_rows_are_multiples_of_eight():
    from exact_b200.dist import shard_rows
    for n, w in ((2449029, 8), (2449029, 2), (100, 4), (7, 2)):
        s = shard_rows(n, w)
        assert s % 8 == 0 and s * w >= n and s * (w - 1) < n + 8 * w


# ---- zero-compacted exchange: the CUDA kernels are replaced by their numpy restatement -----------------
def _stub_rows(xdist):
    import oracle

    def mask_count(x, mask, rowcnt):
        m, ro, _ = oracle.rows_compact(x.numpy())
        mask.copy_(torch.from_numpy(m.view(np.int32)))
        rowcnt.copy_(torch.from_numpy(np.diff(ro).astype(np.int32)))

    def compact_write(x, rowoff, vals):
        _, ro, v = oracle.rows_compact(x.numpy())
        assert np.array_equal(ro, rowoff.numpy()[:ro.size])
        vals[:v.size] = torch.from_numpy(v)

    def expand(mask, rowoff, vals, n, K, block_rows, rowoff_stride, vals_stride, out):
        for b in range(n // block_rows):
            ro = rowoff.numpy()[b * rowoff_stride:b * rowoff_stride + block_rows + 1]
            v = vals.numpy()[b * vals_stride:(b + 1) * vals_stride]
            m = mask.numpy()[b * block_rows:(b + 1) * block_rows].view(np.uint32)
            out[b * block_rows:(b + 1) * block_rows] = torch.from_numpy(oracle.rows_expand(m, ro, v, K))

    xdist.ext_rows.mask_count, xdist.ext_rows.compact_write, xdist.ext_rows.expand = mask_count, compact_write, expand


def _gather_worker(rank, world, port, n, K, result_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from exact_b200 import SparseTensor, config
    from exact_b200 import dist as xdist
    _stub_rows(xdist)
    rowptr, col, _ = random_csr(n, n, 4 * n, 3, False)
    row = np.repeat(np.arange(n), np.diff(rowptr))
    full = SparseTensor(row=torch.from_numpy(row), col=torch.from_numpy(col), value=None, sparse_sizes=(n, n),
                        is_sorted=True)
    adj = xdist.shard_graph(full, "mean", rank, world)
    sparse = normal(n, K, 7)
    sparse[np.random.default_rng(8).random((n, K)) < 0.75] = 0.0
    dense = normal(n, K, 9)
    res = {}
    config.compact_gather = True
    res["sparse"] = adj.gather(torch.from_numpy(sparse[adj.row_start:adj.row_end]), "fw").clone()
    res["streak_after_sparse"] = adj._dense_streak.get("fw", 0)
    res["dense"] = adj.gather(torch.from_numpy(dense[adj.row_start:adj.row_end]), "bw").clone()
    res["streak_after_dense"] = adj._dense_streak.get("bw", 0)
    # while the streak lasts the dense route is taken without trying
    res["dense_again"] = adj.gather(torch.from_numpy(dense[adj.row_start:adj.row_end]), "bw").clone()
    res["streak_after_second"] = adj._dense_streak.get("bw", 0)
    config.compact_gather = False
    res["off"] = adj.gather(torch.from_numpy(sparse[adj.row_start:adj.row_end]), "fw").clone()
    config.compact_gather = True
    torch.save(res, os.path.join(result_dir, f"g{rank}.pt"))
    dist.barrier()
    dist.destroy_process_group()


def test_compacted_gather_equals_dense_gather(tmp_path):
    n, K, world = 203, 64, 2        # 203 rows: the last shard is shorter than the first
    port = _free_port()
    mp.spawn(_gather_worker, args=(world, port, n, K, str(tmp_path)), nprocs=world, join=True)
    sparse = normal(n, K, 7)
    sparse[np.random.default_rng(8).random((n, K)) < 0.75] = 0.0
    dense = normal(n, K, 9)
    for r in range(world):
        p = torch.load(os.path.join(tmp_path, f"g{r}.pt"))
        assert np.array_equal(p["sparse"].numpy().view(np.uint32), sparse.view(np.uint32))
        assert np.array_equal(p["off"].numpy(), sparse)
        assert np.array_equal(p["dense"].numpy(), dense) and np.array_equal(p["dense_again"].numpy(), dense)
        assert p["streak_after_sparse"] == 0 and p["streak_after_dense"] == 16 and p["streak_after_second"] == 15


# ---- feature-parallel aggregation with row blocks: the ranks are threads, the peers' buffers shared tensors -----
def _aggregate_on_threads(world, min_slice, K, n, reduce, with_values, transposed, monkeypatch):
    import threading

    from exact_b200 import SparseTensor, config
    from exact_b200 import dist as xdist

    rowptr, col, val = random_csr(n, n, 6 * n, 3, with_values)
    row = np.repeat(np.arange(n), np.diff(rowptr))
    full = SparseTensor(row=torch.from_numpy(row), col=torch.from_numpy(col),
                        value=None if val is None else torch.from_numpy(val), sparse_sizes=(n, n), is_sorted=True)
    shared, lock, barrier = {}, threading.Lock(), threading.Barrier(world)

    class Buf:
        def __init__(self, tensors, rank):
            self.ptrs, self.rank = tensors, rank

        def local_tensor(self):
            return self.ptrs[self.rank]

    def column_buffers(self, kind, width, nbytes, device):
        key = (kind, width)
        turn = self._col_turn.get(key, 0)
        self._col_turn[key] = turn + 1
        self._col_bufs[key] = True
        with lock:
            tensors = shared.setdefault((kind, width, turn & 1), [torch.full((nbytes // 4,), float("nan")) for _ in range(world)])
        return Buf(tensors, self.rank)

    def cols_scatter(x, rowscale, row0, Kp, dsts):
        m, Kx = x.shape
        xs = x if rowscale is None else x * rowscale.reshape(-1, 1)
        for q, d in enumerate(dsts):
            piece = torch.zeros(m, Kp)
            part = xs[:, q * Kp:(q + 1) * Kp]
            piece[:, :part.size(1)] = part
            d.view(-1, Kp)[row0:row0 + m] = piece

    def rows_scatter(y, shard, col0, ldd, dsts):
        assert y.size(0) <= shard * len(dsts)
        for p, d in enumerate(dsts):
            rows = y[p * shard:(p + 1) * shard]
            d.view(-1, ldd)[:rows.size(0), col0:col0 + y.size(1)] = rows

    def spmm(rowptr, col, value, mat, reduce, regroup=False, route=None):
        assert route is None
        return _oracle_spmm(rowptr, col, value, mat, reduce)

    monkeypatch.setattr(xdist.ShardedSparseTensor, "_column_buffers", column_buffers)
    monkeypatch.setattr(xdist.ShardedSparseTensor, "_order_peer_stores", lambda self, dev: barrier.wait(timeout=60))
    monkeypatch.setattr(xdist.ext_rows, "cols_scatter", cols_scatter)
    monkeypatch.setattr(xdist.ext_rows, "rows_scatter", rows_scatter)
    monkeypatch.setattr(xdist.ext_spmm, "_spmm", spmm)
    monkeypatch.setattr(config, "column_split_aggregation", True)
    monkeypatch.setattr(config, "aggregation_min_slice_columns", min_slice)
    x_full = torch.from_numpy(normal(n, K, 4))
    scale_full = torch.from_numpy(np.abs(normal(n, 1, 6)).reshape(-1) + 0.5)
    outs, errors, slices = [None] * world, [], set()

    def rank_main(r):
        try:
            adj = xdist.ShardedSparseTensor(full, reduce, r, world)
            slices.add(adj.column_slices(K))
            x = x_full[adj.row_start:adj.row_end].clone()
            for _ in range(3):          # three calls: both buffers of a pair are reused
                if transposed:
                    out = adj.aggregate(x, reduce, transposed=True, rowscale=scale_full[adj.row_start:adj.row_end].clone())
                else:
                    out = adj.aggregate(x, reduce)
                outs[r] = out.clone()
        except Exception as e:   # noqa: BLE001
            errors.append((r, repr(e)))
            barrier.abort()

    threads = [threading.Thread(target=rank_main, args=(r,)) for r in range(world)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    assert not errors, errors
    import oracle
    if transposed:
        t_ptr, t_col, _ = full.storage.transposed("sum")
        ref = oracle.spmm(t_ptr.numpy().astype(np.int64), t_col.numpy().astype(np.int64), None,
                          (x_full * scale_full.reshape(-1, 1)).numpy(), "sum")
    else:
        ref = oracle.spmm(rowptr, col, val, x_full.numpy(), reduce)
    got = torch.cat(outs).numpy()
    assert got.shape == ref.shape and np.array_equal(got, ref)
    return slices


def test_feature_parallel_aggregation_row_blocks_on_cpu(monkeypatch):
    # 203 rows on 8 ranks: shards of 32 rows, the last rank's shard is empty, the last row block is short
    assert _aggregate_on_threads(8, 0, 48, 203, "mean", False, False, monkeypatch) == {8}
    assert _aggregate_on_threads(8, 20, 48, 203, "mean", False, False, monkeypatch) == {2}
    assert _aggregate_on_threads(8, 20, 100, 203, "sum", True, False, monkeypatch) == {4}
    assert _aggregate_on_threads(8, 20, 48, 203, "mean", False, True, monkeypatch) == {2}
    assert _aggregate_on_threads(8, 64, 48, 203, "mean", False, False, monkeypatch) == {1}
    assert _aggregate_on_threads(4, 20, 48, 1000, "mean", False, True, monkeypatch) == {2}
