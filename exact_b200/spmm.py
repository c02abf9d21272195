"""QMatmul / qmatmul: sparse-adjacency x dense aggregation that saves its dense operand compressed.
Mirrors exact/exact/spmm.py:7-89 for reduce in {sum, add, mean}."""
import torch
import torch.nn.functional as F
from torch.autograd.function import Function

from .conf import config
from .cpp_extension import spmm as ext_spmm
from .ops import linear_backward_from_compressed, project_and_quantize, qspmm_mean, qspmm_sum
from .qscheme import QScheme
from .utils import empty_cache


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


def _aggregate(src, other, reduce):
    """reduce(A, other) with nothing recorded for backward."""
    from .dist import ShardedSparseTensor, sharded_spmm
    if isinstance(src, ShardedSparseTensor):
        return ext_spmm._spmm(src.rowptr, src.col, src.value, sharded_spmm.gathered_operand(src, other), reduce)
    rowptr, col, value = src.csr()
    return ext_spmm._spmm(rowptr, col, value, other, reduce)


def _aggregate_transposed(src, grad, reduce):
    """Gradient of reduce(A, other) with respect to `other` (spmm.cc:70-77, 128-137)."""
    from .dist import ShardedSparseTensor
    if isinstance(src, ShardedSparseTensor):
        return ext_spmm._spmm(src.t_rowptr, src.t_col, src.t_w, src.gather(grad, "bw"), "sum")
    t_ptr, t_col, t_w = src.storage.transposed(reduce)
    return ext_spmm._spmm(t_ptr, t_col, t_w, grad, "sum")


class qaggregate_linear(Function):
    """y = reduce(A, x) W^T + b, the aggregation + lin_l pair of QSAGEConv (layers.py:163-166), as one
    autograd node.  Forward and the saved compressed tensors are those of QMatmul followed by QLinear.
    Backward uses A^T (g W) = (A^T g) W: the transposed aggregation (and, row-sharded, the gradient
    all-gather before it) runs on the out_features columns of g instead of the in_features columns of
    g W.  It is taken when out_features < in_features; the result differs from the two-node order by
    fp32 reassociation only."""

    @staticmethod
    def forward(ctx, src, x, weight, bias, reduce, lin_scheme):
        agg = _aggregate(src, x, reduce)
        quantized, randmat, proj_shape = project_and_quantize(agg, lin_scheme, True)
        empty_cache(config.empty_cache_threshold)
        ctx.src, ctx.reduce = src, reduce
        ctx.saved = quantized, weight, bias, randmat
        ctx.other_args = agg.shape, proj_shape
        return F.linear(agg, weight, bias)

    @staticmethod
    def backward(ctx, grad_output):
        quantized, weight, bias, randmat = ctx.saved
        ori_shape, proj_shape = ctx.other_args
        del ctx.saved
        grad_output = grad_output.contiguous()
        _, grad_weight, grad_bias = linear_backward_from_compressed(
            quantized, weight, bias, randmat, ori_shape, proj_shape, True, grad_output, False)
        grad_x = None
        if ctx.needs_input_grad[1]:
            out_f = grad_output.size(1)
            pad = (-out_f) % 4   # whole 128-bit column groups for the gather
            if pad:
                g = grad_output.new_zeros((grad_output.size(0), out_f + pad))
                g[:, :out_f].copy_(grad_output)
                w = weight.new_zeros((out_f + pad, weight.size(1)))
                w[:out_f].copy_(weight)
            else:
                g, w = grad_output, weight
            grad_x = _aggregate_transposed(ctx.src, g, ctx.reduce).mm(w)
        return None, grad_x, grad_weight, grad_bias, None, None


def aggregate_linear_applies(src, x, weight):
    """Whether the one-node aggregation + linear is taken: dense-operand gradient wanted, fewer output
    than input features, no edge-value gradient, and the aggregation's own compressed copy (which only
    the edge-value gradient reads) not being kept."""
    from .dist import ShardedSparseTensor
    if not (config.aggregate_gradient_first and config.skip_dead_saves and x.requires_grad):
        return False
    if weight.size(0) >= weight.size(1):
        return False
    if isinstance(src, ShardedSparseTensor):
        return True
    value = src.storage.value()
    return value is None or not value.requires_grad
