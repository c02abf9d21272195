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
