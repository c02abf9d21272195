"""Stand-in for the reference's `exact.cpp_extension.spmm` module (exact/exact/cpp_extension/spmm.cc:243-252):
spmm_{sum,mean}_{fw,bw} with the reference's argument lists, forwarded to the C ABI."""
import ctypes
import weakref

import torch

from .. import _lib
from ..conf import config

_PLANS = {}  # id(rowptr tensor) -> (weak reference to it, {threshold: plan or None})


def _plans_of(rowptr):
    key = id(rowptr)
    hit = _PLANS.get(key)
    if hit is not None and hit[0]() is rowptr:
        return hit[1]
    per = {}
    _PLANS[key] = (weakref.ref(rowptr, lambda _r, k=key: _PLANS.pop(k, None)), per)
    return per


def long_row_plan(rowptr, threshold, col=None):
    """Pieces of the rows with more than `threshold` edges (see exact_spmm_split in the header), built
    once per row-pointer tensor with torch ops and cached.  None when there is no such row.  With `col`
    the pieces are listed by the column of their first edge (item_slot keeps their place in the row):
    pieces of different hub rows that gather the same source rows then run together."""
    per = _plans_of(rowptr)
    key = (threshold, col is not None)
    if key in per:
        return per[key]
    rp = rowptr.to(torch.int64)
    deg = rp[1:] - rp[:-1]
    long_row = torch.nonzero(deg > threshold).flatten()
    plan = None
    if long_row.numel() > 0:
        pieces = (deg[long_row] + threshold - 1) // threshold
        ptr = torch.zeros(long_row.numel() + 1, dtype=torch.int64, device=rowptr.device)
        torch.cumsum(pieces, 0, out=ptr[1:])
        item_row = torch.repeat_interleave(long_row, pieces)
        within = torch.arange(item_row.numel(), device=rowptr.device) - torch.repeat_interleave(ptr[:-1], pieces)
        begin = rp[item_row] + within * threshold
        end = torch.minimum(begin + threshold, rp[item_row + 1])
        slot = None
        if col is not None:
            order = torch.argsort(col[begin].to(torch.int64), stable=True)
            item_row, begin, end = item_row[order], begin[order], end[order]
            slot = order.to(torch.int32).contiguous()
        plan = {"long_row": long_row.to(torch.int32), "long_item_ptr": ptr.to(torch.int32),
                "item_row": item_row.to(torch.int32).contiguous(), "item_begin": begin.contiguous(),
                "item_end": end.contiguous(), "item_slot": slot,
                "n_items": int(item_row.numel()), "n_long": int(long_row.numel())}
    per[key] = plan
    return plan


REGROUP = 0x100   # EXACT_SPMM_REGROUP


def row_order(rowptr):
    """Rows sorted by length (longest first), int32, cached per row-pointer tensor: the order in which the
    kernel for narrow operands takes the rows, so that the rows a warp works on together are equally long."""
    per = _plans_of(rowptr)
    if "row_order" not in per:
        rp = rowptr.to(torch.int64)
        per["row_order"] = torch.argsort(rp[1:] - rp[:-1], stable=True, descending=True).to(torch.int32).contiguous()
    return per["row_order"]


def _spmm(rowptr, col, value, mat, reduce, regroup=False, route=None):
    """spmm.cc:12-18 -> spmm_cuda.cu:106-170.  `regroup`: the caller accepts a regrouped per-row fp32 sum
    (narrow operands then gather several edges per load instruction).  `route` = (shard, col0, ldd, addresses):
    no local result; row r goes to columns col0 .. of row r % shard of the [shard, ldd] buffer at
    addresses[r // shard] (the owners' buffers of a row-sharded run) and None is returned."""
    if not rowptr.is_cuda or not col.is_cuda or not mat.is_cuda:
        raise RuntimeError("rowptr, col and mat must be CUDA tensors")
    if rowptr.dim() != 1 or col.dim() != 1:
        raise RuntimeError("Input mismatch")
    if value is not None and (value.dim() != 1 or value.size(0) != col.size(0)):
        raise RuntimeError("Input mismatch")
    if mat.dim() != 2:
        raise RuntimeError("mat must be [N, K] (batched operands are not used by the GCN/SAGE layers)")
    if mat.dtype not in (torch.float32, torch.float16):
        raise RuntimeError("mat must be float32 or float16")
    if rowptr.dtype != col.dtype or col.dtype not in (torch.int32, torch.int64):
        raise RuntimeError("rowptr and col must both be int32 or both int64")
    mat = mat.contiguous()
    rowptr = rowptr.contiguous()
    col = col.contiguous()
    if mat.dtype == torch.float16:
        # the reference's half instantiation (spmm_cuda.cu:142): every step rounded to half, rows in CSR order
        if route is not None:
            raise RuntimeError("fp16 operands have no routed output")
        if value is not None:
            value = value.detach().to(torch.float16).contiguous()
        M, K = rowptr.numel() - 1, mat.size(1)
        out = torch.empty((M, K), dtype=torch.float16, device=mat.device)
        ib = 4 if col.dtype == torch.int32 else 8
        nnz = col.numel()
        _lib.invoke("exact_spmm_f16", nnz * (2 * K + ib) + 2 * M * K, _lib.ptr(rowptr), _lib.ptr(col), ib, _lib.ptr(value),
                    _lib.ptr(mat), M, K, _lib.REDUCE[reduce], _lib.ptr(out), _lib.stream_ptr())
        return out
    if value is not None:
        value = value.detach().to(torch.float32).contiguous()
    M = rowptr.numel() - 1
    K = mat.size(1)
    out = torch.empty((M, K), dtype=mat.dtype, device=mat.device) if route is None else None
    ib = 4 if col.dtype == torch.int32 else 8
    nnz = col.numel()
    index_bytes = nnz * (ib + (4 if value is not None else 0)) + (M + 1) * ib
    # bytes that must cross HBM at least once (operand, indices, output), and the bytes the gathers request
    # from L2 when no source row is reused (what the reference's kernel moves)
    nbytes = mat.size(0) * K * 4 + index_bytes + M * K * 4
    l2_bytes = nnz * K * 4 + index_bytes + M * K * 4
    thr = int(config.spmm_long_row)
    plan = long_row_plan(rowptr, thr, col) if thr > 0 else None
    red = _lib.REDUCE[reduce] | (REGROUP if regroup else 0)
    narrow = K <= 64 and K % 4 == 0 and M > 0
    if route is None and narrow:
        route = (M, 0, K, [out.data_ptr()])   # the same entry point, one local destination: it takes a row order
    if route is not None:
        shard, col0, ldd, addresses = route
        arr = (ctypes.c_void_p * len(addresses))(*addresses)
        order = row_order(rowptr) if narrow else None
        none = {"item_row": None, "item_begin": None, "item_end": None, "item_slot": None, "n_items": 0,
                "long_row": None, "long_item_ptr": None, "n_long": 0}
        pl = plan if plan is not None else none
        scratch = torch.empty((pl["n_items"], K), dtype=torch.float32, device=mat.device) if plan is not None else None
        _lib.invoke("exact_spmm_split_routed", nbytes, _lib.ptr(rowptr), _lib.ptr(col), ib, _lib.ptr(value),
                    _lib.ptr(mat), M, K, red, thr if plan is not None else 0, _lib.ptr(pl["item_row"]),
                    _lib.ptr(pl["item_begin"]), _lib.ptr(pl["item_end"]), _lib.ptr(pl["item_slot"]), pl["n_items"],
                    _lib.ptr(pl["long_row"]), _lib.ptr(pl["long_item_ptr"]), pl["n_long"], _lib.ptr(scratch),
                    _lib.ptr(order), shard, col0, ldd, arr, len(addresses), _lib.stream_ptr(), device=mat.device,
                    l2_bytes=l2_bytes, edge_columns=nnz * K)
        return out
    if plan is None:
        _lib.invoke("exact_spmm", nbytes, _lib.ptr(rowptr), _lib.ptr(col), ib, _lib.ptr(value), _lib.ptr(mat), M, K,
                    red, _lib.ptr(out), _lib.stream_ptr(), l2_bytes=l2_bytes, edge_columns=nnz * K)
    else:
        scratch = torch.empty((plan["n_items"], K), dtype=torch.float32, device=mat.device)
        _lib.invoke("exact_spmm_split", nbytes, _lib.ptr(rowptr), _lib.ptr(col), ib, _lib.ptr(value), _lib.ptr(mat),
                    M, K, red, thr, _lib.ptr(plan["item_row"]), _lib.ptr(plan["item_begin"]),
                    _lib.ptr(plan["item_end"]), _lib.ptr(plan["item_slot"]), plan["n_items"], _lib.ptr(plan["long_row"]),
                    _lib.ptr(plan["long_item_ptr"]), plan["n_long"], _lib.ptr(scratch), _lib.ptr(out),
                    _lib.stream_ptr(), l2_bytes=l2_bytes, edge_columns=nnz * K)
    return out


def spmm_sum_fw(row, rowptr, col, value, colptr, csr2csc, mat):
    """spmm.cc:31-55."""
    return _spmm(rowptr, col, value, mat, "sum")


def spmm_mean_fw(row, rowptr, col, value, rowcount, colptr, csr2csc, mat):
    """spmm.cc:84-113."""
    return _spmm(rowptr, col, value, mat, "mean")


def spmm_value_bw(row, rowptr, col, mat, grad, reduce):
    """spmm.cc:20-24 -> spmm_cuda.cu:211-252: gradient with respect to the edge values, [nnz] fp32."""
    if not (row.is_cuda and col.is_cuda and mat.is_cuda and grad.is_cuda):
        raise RuntimeError("row, col, mat and grad must be CUDA tensors")
    if mat.dtype != torch.float32 or grad.dtype != torch.float32 or mat.dim() != 2 or grad.dim() != 2:
        raise RuntimeError("mat and grad must be float32 matrices")
    if not (row.dtype == col.dtype == rowptr.dtype) or col.dtype not in (torch.int32, torch.int64):
        raise RuntimeError("row, rowptr and col must all be int32 or all int64")
    mat, grad = mat.contiguous(), grad.contiguous()
    row, col, rowptr = row.contiguous(), col.contiguous(), rowptr.contiguous()
    E, K = col.numel(), mat.size(1)
    out = torch.empty(E, dtype=torch.float32, device=mat.device)
    ib = 4 if col.dtype == torch.int32 else 8
    _lib.invoke("exact_spmm_value_bw", E * (8 * K + 2 * ib + 4), _lib.ptr(row), _lib.ptr(rowptr), _lib.ptr(col), ib,
                _lib.ptr(mat), _lib.ptr(grad), E, K, _lib.REDUCE[reduce], _lib.ptr(out), _lib.stream_ptr())
    return out


def spmm_sum_bw(row, rowptr, col, value, colptr, csr2csc, mat, grad_out, has_value, value_requires_grad,
                mat_requires_grad, transposed=None):
    """spmm.cc:57-79.  `transposed` = (colptr, row[csr2csc], value[csr2csc]) when the caller caches it."""
    grad_value = None
    if has_value and value_requires_grad:
        grad_value = spmm_value_bw(row, rowptr, col, mat, grad_out, "sum")
    grad_mat = None
    if mat_requires_grad:
        if transposed is None:
            w = value.index_select(0, csr2csc) if has_value else None
            transposed = (colptr, row.index_select(0, csr2csc), w)
        grad_mat = _spmm(transposed[0], transposed[1], transposed[2], grad_out, "sum")
    return grad_value, grad_mat


def spmm_mean_bw(row, rowptr, col, value, rowcount, colptr, csr2csc, mat, grad_out, has_value,
                 value_requires_grad, mat_requires_grad, transposed=None):
    """spmm.cc:115-139."""
    grad_value = None
    if has_value and value_requires_grad:
        grad_value = spmm_value_bw(row, rowptr, col, mat, grad_out, "mean")
    grad_mat = None
    if mat_requires_grad:
        if transposed is None:
            row_t = row.index_select(0, csr2csc)
            cnt = rowcount.to(grad_out.dtype).index_select(0, row_t.to(torch.int64)).clamp_(1)
            w = value.index_select(0, csr2csc).div(cnt) if has_value else cnt.pow_(-1)
            transposed = (colptr, row_t, w)
        grad_mat = _spmm(transposed[0], transposed[1], transposed[2], grad_out, "sum")
    return grad_value, grad_mat


def _spmm_minmax(rowptr, col, value, mat, is_max):
    if not (rowptr.is_cuda and col.is_cuda and mat.is_cuda):
        raise RuntimeError("rowptr, col and mat must be CUDA tensors")
    if mat.dim() != 2 or mat.dtype != torch.float32:
        raise RuntimeError("mat must be a float32 matrix")
    if rowptr.dtype != col.dtype or col.dtype not in (torch.int32, torch.int64):
        raise RuntimeError("rowptr and col must both be int32 or both int64")
    mat, rowptr, col = mat.contiguous(), rowptr.contiguous(), col.contiguous()
    if value is not None:
        value = value.detach().to(torch.float32).contiguous()
    M, K, nnz = rowptr.numel() - 1, mat.size(1), col.numel()
    out = torch.empty((M, K), dtype=torch.float32, device=mat.device)
    arg_out = torch.empty((M, K), dtype=col.dtype, device=mat.device)
    ib = 4 if col.dtype == torch.int32 else 8
    _lib.invoke("exact_spmm_minmax", nnz * (K * 4 + ib) + M * K * (4 + ib), _lib.ptr(rowptr), _lib.ptr(col), ib,
                _lib.ptr(value), _lib.ptr(mat), M, K, nnz, 1 if is_max else 0, _lib.ptr(out), _lib.ptr(arg_out),
                _lib.stream_ptr())
    return out, arg_out


def spmm_max_fw(rowptr, col, value, mat):
    """spmm.cc:145-157 -> (out, arg_out)."""
    return _spmm_minmax(rowptr, col, value, mat, True)


def spmm_min_fw(rowptr, col, value, mat):
    """spmm.cc:195-208 -> (out, arg_out)."""
    return _spmm_minmax(rowptr, col, value, mat, False)


def spmm_max_bw(col, value, mat, arg_out, grad_out, has_value, value_requires_grad, mat_requires_grad):
    """spmm.cc:159-193 (and 210-241 for min, the same arithmetic): gradients routed to the winning edges."""
    arg_out = arg_out.to(torch.int64)
    invalid = arg_out == col.size(0)
    arg_out = arg_out.masked_fill(invalid, 0)
    ind = col.to(torch.int64).index_select(0, arg_out.flatten()).view_as(arg_out)
    grad_value = None
    if has_value and value_requires_grad:
        out = mat.gather(-2, ind)
        out.mul_(grad_out)
        out.masked_fill_(invalid, 0)
        grad_value = torch.zeros_like(value)
        grad_value.scatter_add_(0, arg_out.flatten(), out.flatten())
    grad_mat = None
    if mat_requires_grad:
        if has_value:
            v = value.detach().index_select(0, arg_out.flatten()).view_as(arg_out)
            v = v * grad_out
        else:
            v = grad_out.clone()
        v.masked_fill_(invalid, 0)
        grad_mat = torch.zeros_like(mat)
        grad_mat.scatter_add_(-2, ind, v)
    return grad_value, grad_mat


spmm_min_bw = spmm_max_bw
