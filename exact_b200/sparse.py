"""A CSR adjacency container with the slice of torch_sparse.SparseTensor's interface that the
reference touches (exact/exact/spmm.py:18-44: csr(), storage._row/_rowcount/_colptr/_csr2csc and their
computing accessors; mem_speed_bench drivers: set_diag, gcn_norm, fill_cache_, to/cuda).

torch_sparse is not a dependency.  Extra to the reference: the transposed structure needed by the
SpMM backward (spmm.cc:70-77, 128-137 rebuild it with index_select on every call) is computed once and
cached here.
"""
import torch


class SparseStorage:
    def __init__(self, row, rowptr, col, value, sparse_sizes):
        self._row = row
        self._rowptr = rowptr
        self._col = col
        self._value = value
        self._sparse_sizes = tuple(sparse_sizes)
        self._rowcount = None
        self._colptr = None
        self._csr2csc = None
        self._t_cache = {}

    # -- computing accessors (torch_sparse.storage semantics) --
    def row(self):
        if self._row is None:
            M = self._sparse_sizes[0]
            counts = self.rowcount().to(torch.int64)
            self._row = torch.repeat_interleave(
                torch.arange(M, device=self._col.device, dtype=self._col.dtype), counts)
        return self._row

    def rowptr(self):
        return self._rowptr

    def col(self):
        return self._col

    def value(self):
        return self._value

    def rowcount(self):
        if self._rowcount is None:
            self._rowcount = self._rowptr[1:] - self._rowptr[:-1]
        return self._rowcount

    def csr2csc(self):
        if self._csr2csc is None:
            key = self._col.to(torch.int64) * self._sparse_sizes[0] + self.row().to(torch.int64)
            self._csr2csc = torch.argsort(key, stable=True)
        return self._csr2csc

    def colptr(self):
        if self._colptr is None:
            N = self._sparse_sizes[1]
            counts = torch.bincount(self._col.to(torch.int64), minlength=N)
            colptr = torch.zeros(N + 1, dtype=self._rowptr.dtype, device=self._col.device)
            torch.cumsum(counts, 0, out=colptr[1:])
            self._colptr = colptr
        return self._colptr

    def sparse_sizes(self):
        return self._sparse_sizes

    # -- transposed structure for the dense-operand gradient, cached --
    def transposed(self, reduce):
        """(colptr, row[csr2csc], weights) with weights = value[csr2csc] (sum; None without values)
        or value[csr2csc] / clamp(rowcount[row], 1) (mean), as spmm.cc:70-77 / 128-137 build them."""
        version = None if self._value is None else self._value._version
        hit = self._t_cache.get(reduce)
        if hit is not None and hit[0] == version:
            return hit[1]
        perm = self.csr2csc()
        row_t = self.row().index_select(0, perm).contiguous()
        if reduce == "mean":
            cnt = self.rowcount().to(torch.float32).index_select(0, row_t.to(torch.int64)).clamp_(1)
            if self._value is not None:
                w = self._value.detach().index_select(0, perm).div(cnt)
            else:
                w = cnt.pow_(-1)
        else:
            w = None if self._value is None else self._value.detach().index_select(0, perm).contiguous()
        out = (self.colptr(), row_t, w)
        self._t_cache[reduce] = (version, out)
        return out


class SparseTensor:
    def __init__(self, row=None, rowptr=None, col=None, value=None, sparse_sizes=None, is_sorted=False):
        assert col is not None and sparse_sizes is not None
        if rowptr is None:
            assert row is not None
            if not is_sorted:
                key = row.to(torch.int64) * sparse_sizes[1] + col.to(torch.int64)
                perm = torch.argsort(key, stable=True)
                row, col = row[perm], col[perm]
                if value is not None:
                    value = value[perm]
            counts = torch.bincount(row.to(torch.int64), minlength=sparse_sizes[0])
            rowptr = torch.zeros(sparse_sizes[0] + 1, dtype=col.dtype, device=col.device)
            torch.cumsum(counts, 0, out=rowptr[1:])
        self.storage = SparseStorage(row, rowptr.contiguous(), col.contiguous(),
                                     None if value is None else value.contiguous(), sparse_sizes)

    @classmethod
    def from_edge_index(cls, edge_index, edge_attr=None, sparse_sizes=None, is_sorted=False):
        row, col = edge_index[0], edge_index[1]
        if sparse_sizes is None:
            n = int(max(int(row.max()), int(col.max()))) + 1
            sparse_sizes = (n, n)
        return cls(row=row, col=col, value=edge_attr, sparse_sizes=tuple(sparse_sizes), is_sorted=is_sorted)

    # -- torch_sparse-like surface --
    def csr(self):
        s = self.storage
        return s._rowptr, s._col, s._value

    def coo(self):
        s = self.storage
        return s.row(), s._col, s._value

    def sparse_sizes(self):
        return self.storage._sparse_sizes

    def size(self, dim):
        return self.storage._sparse_sizes[dim]

    def nnz(self):
        return self.storage._col.numel()

    @property
    def device(self):
        return self.storage._col.device

    def has_value(self):
        return self.storage._value is not None

    def set_value(self, value, layout=None):
        s = self.storage
        out = SparseTensor(row=s._row, rowptr=s._rowptr, col=s._col, value=value, sparse_sizes=s._sparse_sizes)
        out.storage._rowcount, out.storage._colptr, out.storage._csr2csc = s._rowcount, s._colptr, s._csr2csc
        return out

    def fill_cache_(self):
        s = self.storage
        s.row(); s.rowcount(); s.colptr(); s.csr2csc()
        return self

    def set_diag(self, fill_value=1.0):
        """Drop existing diagonal entries and add one per node (torch_sparse.set_diag)."""
        row, col, value = self.coo()
        M, N = self.sparse_sizes()
        keep = row != col
        n = min(M, N)
        loop = torch.arange(n, device=col.device, dtype=col.dtype)
        new_row = torch.cat([row[keep], loop])
        new_col = torch.cat([col[keep], loop])
        new_val = None
        if value is not None:
            new_val = torch.cat([value[keep], torch.full((n,), fill_value, dtype=value.dtype, device=value.device)])
        return SparseTensor(row=new_row, col=new_col, value=new_val, sparse_sizes=(M, N))

    def t(self):
        row, col, value = self.coo()
        M, N = self.sparse_sizes()
        return SparseTensor(row=col, col=row, value=value, sparse_sizes=(N, M))

    def _map(self, fn, value_fn=None):
        s = self.storage
        value_fn = value_fn or fn
        out = SparseTensor(row=None if s._row is None else fn(s._row), rowptr=fn(s._rowptr), col=fn(s._col),
                           value=None if s._value is None else value_fn(s._value), sparse_sizes=s._sparse_sizes)
        for name in ("_rowcount", "_colptr", "_csr2csc"):
            v = getattr(s, name)
            setattr(out.storage, name, None if v is None else fn(v))
        return out

    def to(self, device):
        return self._map(lambda t: t.to(device))

    def cuda(self, device=None):
        return self.to("cuda" if device is None else device)

    def cpu(self):
        return self.to("cpu")

    def to_int32_(self):
        """Narrow index arrays to int32 in place (the reference's cast_adj, utils.py:22-28)."""
        s = self.storage
        assert self.nnz() < 2**31 - 1 and max(s._sparse_sizes) < 2**31 - 1
        for name in ("_row", "_rowptr", "_col", "_rowcount", "_colptr", "_csr2csc"):
            v = getattr(s, name)
            if v is not None:
                setattr(s, name, v.to(torch.int32))
        s._t_cache = {}
        return self

    def to_dense(self):
        row, col, value = self.coo()
        M, N = self.sparse_sizes()
        out = torch.zeros(M, N, dtype=torch.float32 if value is None else value.dtype, device=col.device)
        v = torch.ones(col.numel(), dtype=out.dtype, device=col.device) if value is None else value
        out.index_put_((row.to(torch.int64), col.to(torch.int64)), v, accumulate=True)
        return out


def gcn_norm(adj_t, add_self_loops=True):
    """D^-1/2 (A [+ I]) D^-1/2 on a SparseTensor (torch_geometric.nn.conv.gcn_conv.gcn_norm, the
    SparseTensor branch the drivers call: mem_speed_bench/arxiv/train_full_batch.py:192-196)."""
    if not adj_t.has_value():
        adj_t = adj_t.set_value(torch.ones(adj_t.nnz(), dtype=torch.float32, device=adj_t.device))
    if add_self_loops:
        adj_t = adj_t.set_diag(1.0)
    row, col, value = adj_t.coo()
    M = adj_t.size(0)
    deg = torch.zeros(M, dtype=value.dtype, device=value.device).index_add_(0, row.to(torch.int64), value)
    dis = deg.pow(-0.5)
    dis.masked_fill_(dis == float("inf"), 0.0)
    value = dis[row.to(torch.int64)] * value * dis[col.to(torch.int64)]
    return adj_t.set_value(value)
