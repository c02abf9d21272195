"""The scratch-free variant of the long-row SpMM, for hosts that cannot allocate device memory.

Some callers of this library run where a cudaMalloc is not allowed at call time: an inference server
whose device memory was planned and frozen at start-up, an operator embedded in another runtime that
owns the allocator, code between the begin and end of a recorded region.  exact_spmm_split_static
serves them: its partial-sum buffer is a fixed 16 MiB array inside the library.  This test calls it
through the C ABI twice in a row and requires bit-identical output to exact_spmm_split (which takes a
caller-owned buffer), and checks that a plan larger than the built-in array is refused.

Collected last on purpose (file name), so that a failure here cannot hide another test's result."""
import numpy as np
import pytest
import torch

from exact_b200 import _lib
from exact_b200.cpp_extension import spmm as S

pytestmark = pytest.mark.gpu


def _graph(n, seed):
    rng = np.random.default_rng(seed)
    hubs = [np.stack([np.full(d, r, np.int64), rng.choice(n, d, replace=False)])
            for r, d in ((5, 3000), (1234, 900), (n - 1, 1500))]
    rest = rng.integers(0, n, (2, 40000))
    e = np.concatenate(hubs + [rest], 1)
    key = np.unique(e[0] * n + e[1])
    row, col = key // n, key % n
    rowptr = np.zeros(n + 1, np.int64)
    np.cumsum(np.bincount(row, minlength=n), out=rowptr[1:])
    return rowptr, col


def _call(name, rowptr, col, val, mat, reduce, thr, plan, scratch, out):
    lib = _lib.load()
    args = [_lib.ptr(rowptr), _lib.ptr(col), 8, _lib.ptr(val), _lib.ptr(mat), rowptr.numel() - 1, mat.size(1),
            _lib.REDUCE[reduce], thr, _lib.ptr(plan["item_row"]), _lib.ptr(plan["item_begin"]),
            _lib.ptr(plan["item_end"]), _lib.ptr(plan.get("item_slot")), plan["n_items"], _lib.ptr(plan["long_row"]),
            _lib.ptr(plan["long_item_ptr"]),
            plan["n_long"]]
    if scratch is not None:
        args.append(_lib.ptr(scratch))
    args += [_lib.ptr(out), torch.cuda.current_stream().cuda_stream]
    return getattr(lib, name)(*args)


@pytest.mark.parametrize("reduce", ["sum", "mean"])
def test_static_scratch_matches_caller_scratch_twice(reduce):
    n, K, thr = 5000, 128, 512
    rowptr_np, col_np = _graph(n, 1)
    rowptr, col = torch.from_numpy(rowptr_np).cuda(), torch.from_numpy(col_np).cuda()
    plan = S.long_row_plan(rowptr, thr, col)   # pieces listed by first column, slots by place in the row
    assert plan is not None and plan["n_long"] == 3 and plan["n_items"] * K <= 4 * 1024 * 1024
    for rep in range(2):   # two calls in a row share the built-in array
        g = torch.Generator(device="cuda").manual_seed(10 + rep)
        mat = torch.randn(n, K, device="cuda", generator=g)
        val = torch.randn(col.numel(), device="cuda", generator=g)
        ref = torch.empty(n, K, device="cuda")
        scratch = torch.empty(plan["n_items"], K, device="cuda")
        assert _call("exact_spmm_split", rowptr, col, val, mat, reduce, thr, plan, scratch, ref) == 0
        out = torch.full((n, K), float("nan"), device="cuda")
        before = torch.cuda.memory_allocated()
        assert _call("exact_spmm_split_static", rowptr, col, val, mat, reduce, thr, plan, None, out) == 0
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before
        assert torch.equal(out, ref)   # same kernels, same order: bit-identical


def test_plan_larger_than_the_builtin_array_is_refused():
    n, K, thr = 5000, 128, 512
    rowptr_np, col_np = _graph(n, 2)
    rowptr, col = torch.from_numpy(rowptr_np).cuda(), torch.from_numpy(col_np).cuda()
    plan = dict(S.long_row_plan(rowptr, thr))
    mat = torch.randn(n, K, device="cuda")
    out = torch.empty(n, K, device="cuda")
    plan["n_items"] = 4 * 1024 * 1024 // K + 1    # one slice more than the array holds
    rc = _call("exact_spmm_split_static", rowptr, col, None, mat, "sum", thr, plan, None, out)
    assert rc == 1 and b"built-in scratch array" in _lib.load().exact_last_error()
