"""Zero-compacted rows (exact_rows_*): the exchange format of the row-sharded aggregation.  The
reference is single-GPU and has no counterpart."""
import torch

from .. import _lib


def _check(x):
    if not (x.is_cuda and x.dtype == torch.float32 and x.dim() == 2 and x.stride(1) == 1):
        raise RuntimeError("rows: expected a CUDA fp32 matrix with unit column stride")
    if x.size(1) % 32 != 0:
        raise RuntimeError("rows: the number of columns must be a multiple of 32")


def mask_count(x, mask, rowcnt):
    """mask [n, K/32] int32 and rowcnt [n] int32 of x [n, K]."""
    _check(x)
    n, K = x.shape
    assert mask.dtype == torch.int32 and mask.is_contiguous() and mask.numel() == n * (K // 32)
    assert rowcnt.dtype == torch.int32 and rowcnt.is_contiguous() and rowcnt.numel() == n
    _lib.invoke("exact_rows_mask_count", 4 * n * K + n * K // 8 + 4 * n, _lib.ptr(x), n, K, x.stride(0) if n else K,
                _lib.ptr(mask), _lib.ptr(rowcnt), _lib.stream_ptr())


def compact_write(x, rowoff, vals):
    """vals[rowoff[r] ...] = kept elements of row r; rowoff int64 [n + 1]."""
    _check(x)
    n, K = x.shape
    assert rowoff.dtype == torch.int64 and rowoff.is_contiguous() and rowoff.numel() >= n + 1
    assert vals.dtype == torch.float32 and vals.is_contiguous()
    _lib.invoke("exact_rows_compact_write", 4 * n * K + 4 * vals.numel(), _lib.ptr(x), n, K,
                x.stride(0) if n else K, _lib.ptr(rowoff), _lib.ptr(vals), _lib.stream_ptr())


def expand(mask, rowoff, vals, n, K, block_rows, rowoff_stride, vals_stride, out):
    """Dense rows out[:n, :K] from `n / block_rows` compacted shards laid out back to back."""
    assert mask.dtype == torch.int32 and rowoff.dtype == torch.int64 and vals.dtype == torch.float32
    assert out.dtype == torch.float32 and out.stride(1) == 1 and out.size(0) >= n and out.size(1) == K
    _lib.invoke("exact_rows_expand", 4 * n * K + n * K // 8 + 4 * vals.numel(), _lib.ptr(mask), _lib.ptr(rowoff),
                _lib.ptr(vals), n, K, block_rows, rowoff_stride, vals_stride, _lib.ptr(out), out.stride(0),
                _lib.stream_ptr())


def compact(x):
    """(mask, rowoff, vals) of x; synchronises to size vals."""
    n, K = x.shape
    mask = torch.empty((n, K // 32), dtype=torch.int32, device=x.device)
    rowcnt = torch.empty(n, dtype=torch.int32, device=x.device)
    mask_count(x, mask, rowcnt)
    rowoff = torch.zeros(n + 1, dtype=torch.int64, device=x.device)
    torch.cumsum(rowcnt, 0, out=rowoff[1:])
    vals = torch.empty(max(int(rowoff[-1].item()), 1), dtype=torch.float32, device=x.device)
    compact_write(x, rowoff, vals)
    return mask, rowoff, vals
