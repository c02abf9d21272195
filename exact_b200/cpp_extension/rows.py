"""Sparse forms of dense operands that are mostly exact zeros.  The reference is single-GPU, gathers dense
rows and has no counterpart.

Compact rows (exact_crows_*): fixed-size slots holding each row's kept columns and values; what the SpMM
gathers from and what row shards write into each other's memory.  Zero-compacted rows (exact_rows_*):
mask + offsets + values, the wire format of the collective-library exchange."""
import ctypes

import torch

from .. import _lib
from ..conf import config


class CompactRows:
    """`rows` slots of an [rows, K] fp32 matrix in one uint8 buffer (see exact_crows_pack)."""

    def __init__(self, buf, rows, K, density=0.25, address=None, device=None):
        """`buf`: the uint8 tensor that holds the slots, or None with the device `address` of memory owned
        elsewhere (a buffer the library allocated for peers to write into)."""
        self.buf, self.rows, self.K = buf, rows, K
        self.slot_bytes = slot_bytes(K)
        self.density = density     # last measured share of kept entries (byte accounting only)
        self._address = buf.data_ptr() if buf is not None else address
        self._device = buf.device if buf is not None else device

    @property
    def device(self):
        return self._device

    def ptr(self):
        return self._address


class OperandForm:
    """Remembers, per adjacency and call site, whether the dense operand of an aggregation is worth exchanging
    as compact rows.  The first call and every `reprobe`-th one measure the share of non-zero entries (one
    host read of a device counter); the calls between reuse the decision, so the steady state has no
    synchronisation.  Either route delivers the same dense rows bit for bit."""

    reprobe = 64

    def __init__(self):
        self.state = {}     # tag -> [mode, calls until the next probe, last density]

    def mode(self, tag, K, dtype):
        if not (config.compact_operand and dtype == torch.float32 and 64 <= K <= 256 and K % 4 == 0):
            return "dense", 1.0
        st = self.state.get(tag)
        if st is None or st[1] <= 0:
            return "probe", 0.25 if st is None else st[2]
        st[1] -= 1
        return st[0], st[2]

    def decide(self, tag, density):
        mode = "compact" if density <= config.compact_operand_max_density else "dense"
        self.state[tag] = [mode, self.reprobe, density]
        return mode


def slot_bytes(K):
    n = int(_lib.load().exact_crows_slot_bytes(K))
    if n < 0:
        raise RuntimeError(f"compact rows hold at most 256 columns (got {K})")
    return n


def crows_alloc(rows, K, device):
    """An uninitialised buffer of `rows` slots."""
    return CompactRows(torch.empty(rows * slot_bytes(K), dtype=torch.uint8, device=device), rows, K)


def crows_pack(x, rowscale=None, out=None, row0=0, dst_ptrs=None, kept_total=None):
    """Compact rows of x [n, K] (optionally x * rowscale[:, None]) into slots row0 .. row0 + n - 1 of `out`
    (allocated when None) or of every buffer whose device address `dst_ptrs` lists (peers' buffers
    included).  `kept_total`: a one-element int64 device tensor the number of kept entries is added to."""
    if not (x.is_cuda and x.dtype == torch.float32 and x.dim() == 2 and x.stride(1) == 1):
        raise RuntimeError("crows_pack: expected a CUDA fp32 matrix with unit column stride")
    n, K = x.shape
    if out is None and dst_ptrs is None:
        out = crows_alloc(row0 + n, K, x.device)
    if dst_ptrs is None:
        assert out.K == K and out.rows >= row0 + n
        dst_ptrs = [out.ptr()]
    if rowscale is not None:
        rowscale = rowscale.reshape(-1)
        assert rowscale.dtype == torch.float32 and rowscale.numel() == n and rowscale.is_contiguous()
    arr = (ctypes.c_void_p * len(dst_ptrs))(*dst_ptrs)
    nbytes = 4 * n * K + len(dst_ptrs) * n * (16 + K // 4 * 5)   # read once; ~25 % kept, written per destination
    _lib.invoke("exact_crows_pack", nbytes, _lib.ptr(x), n, K, x.stride(0) if n else K, _lib.ptr(rowscale), row0, arr,
                len(dst_ptrs), _lib.ptr(kept_total), _lib.stream_ptr(), device=x.device)
    return out


def crows_unpack(cr, n=None, row0=0, out=None):
    """Dense [n, K] fp32 matrix of slots row0 .. row0 + n - 1 (into the first n rows of `out` when given)."""
    n = cr.rows - row0 if n is None else n
    if out is None:
        out = torch.empty((n, cr.K), dtype=torch.float32, device=cr.device)
    assert out.dtype == torch.float32 and out.size(0) >= n and out.size(1) == cr.K and out.stride(1) == 1
    _lib.invoke("exact_crows_unpack", 4 * n * cr.K + n * (16 + int(cr.density * cr.K) * 5), cr.ptr(), n, cr.K, row0,
                _lib.ptr(out), out.stride(0), _lib.stream_ptr(), device=cr.device)
    return out[:n]


def cols_scatter(x, rowscale, row0, Kp, dst_ptrs):
    """Column slice q of the rows of x [n, K] (times rowscale[:, None]) into rows row0 .. row0 + n - 1 of the
    [*, Kp] buffer at dst_ptrs[q], for every q (first exchange of the feature-parallel aggregation)."""
    n, K = x.shape
    if rowscale is not None:
        rowscale = rowscale.reshape(-1)
        assert rowscale.dtype == torch.float32 and rowscale.numel() == n and rowscale.is_contiguous()
    arr = (ctypes.c_void_p * len(dst_ptrs))(*dst_ptrs)
    _lib.invoke("exact_cols_scatter", 4 * n * K + 4 * n * Kp * len(dst_ptrs), _lib.ptr(x), n, K, x.stride(0) if n else K,
                _lib.ptr(rowscale), row0, Kp, arr, len(dst_ptrs), _lib.stream_ptr(), device=x.device)


def rows_scatter(y, shard, col0, ldd, dst_ptrs):
    """Row block p of y [n_total, Kp] into columns col0 .. col0 + Kp - 1 of the [shard, ldd] buffer at
    dst_ptrs[p], for every p (second exchange of the feature-parallel aggregation)."""
    assert y.dtype == torch.float32 and y.is_contiguous()
    n_total, Kp = y.shape
    arr = (ctypes.c_void_p * len(dst_ptrs))(*dst_ptrs)
    _lib.invoke("exact_rows_scatter", 8 * n_total * Kp, _lib.ptr(y), n_total, Kp, shard, col0, ldd, arr, len(dst_ptrs),
                _lib.stream_ptr(), device=y.device)


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
