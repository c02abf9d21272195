"""QMatmul / qmatmul: sparse-adjacency x dense aggregation that saves its dense operand compressed.
Mirrors exact/exact/spmm.py:7-89 for reduce in {sum, add, mean}."""
import torch

from .conf import config
from .ops import qspmm_mean, qspmm_sum
from .qscheme import QScheme


def qmatmul(src, other, reduce="sum", quantized=None, randmat=None, scheme=None):
    """spmm.py:55-89.  A row-sharded adjacency (exact_b200.dist.ShardedSparseTensor) takes the
    all-gather + local-SpMM route instead."""
    from .dist import ShardedSparseTensor, sharded_spmm
    if isinstance(src, ShardedSparseTensor):
        if reduce in ["sum", "add"]:
            reduce = "sum"
        assert reduce == src.reduce, "the shard was built for a different reduction"
        return sharded_spmm.apply(src, other, reduce)
    rowptr, col, value = src.csr()
    has_value = value is not None
    st = src.storage
    value_rg = has_value and value.requires_grad
    if reduce in ["sum", "add"]:
        row, csr2csc, colptr = st._row, st._csr2csc, st._colptr
        if value_rg:
            row = st.row()
        if other.requires_grad:
            row, csr2csc, colptr = st.row(), st.csr2csc(), st.colptr()
        return qspmm_sum.apply(row, rowptr, col, value, colptr, csr2csc, has_value, other, quantized, randmat,
                               scheme, st)
    elif reduce == "mean":
        row, rowcount, csr2csc, colptr = st._row, st._rowcount, st._csr2csc, st._colptr
        if value_rg:
            row = st.row()
        if other.requires_grad:
            row, rowcount, csr2csc, colptr = st.row(), st.rowcount(), st.csr2csc(), st.colptr()
        return qspmm_mean.apply(row, rowptr, col, value, rowcount, colptr, csr2csc, has_value, other, quantized,
                                randmat, scheme, st)
    elif reduce in ("min", "max"):
        raise NotImplementedError("min/max aggregation is used by neither GCN nor GraphSAGE-mean; "
                                  "only sum and mean are provided")
    raise ValueError(reduce)


class QMatmul(torch.nn.Module):
    """spmm.py:7-52."""

    def __init__(self, reduce):
        super().__init__()
        if reduce in ["sum", "add"]:
            reduce = "sum"
        self.reduce = reduce
        self.scheme = QScheme("matmul") if config.single_precision else None

    def forward(self, src, other, quantized=None, randmat=None):
        return qmatmul(src, other, self.reduce, quantized, randmat, self.scheme)
