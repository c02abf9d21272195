"""QMatmul / qmatmul: sparse-adjacency x dense aggregation that saves its dense operand compressed.
Mirrors exact/exact/spmm.py:7-89 for reduce in {sum, add, mean}."""
import torch
from torch.amp import custom_bwd, custom_fwd
import torch.nn.functional as F
from torch.autograd.function import Function

from .conf import config
from .cpp_extension import backward_func as ext_backward_func
from .cpp_extension import quantization as ext_quantization
from .cpp_extension import spmm as ext_spmm
from .ops import (_rademacher, linear_backward_from_compressed, project_and_quantize, qspmm_max, qspmm_mean, qspmm_min,
                  qspmm_sum)
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
    elif reduce == "min":      # spmm.py:46-48
        return qspmm_min.apply(rowptr, col, value, has_value, other, quantized, randmat, scheme)
    elif reduce == "max":      # spmm.py:49-51
        return qspmm_max.apply(rowptr, col, value, has_value, other, quantized, randmat, scheme)
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


def _operand(src, x, tag, rowscale=None):
    """The dense operand x (times rowscale[:, None]) of an aggregation over `src`, with every row the local
    adjacency rows reference in local HBM."""
    from .dist import ShardedSparseTensor
    if isinstance(src, ShardedSparseTensor):
        return src.exchange(x, tag, rowscale)
    return x if rowscale is None else x * rowscale.unsqueeze(1)


def _aggregate(src, other, reduce, tag="fw", meanwhile=None):
    """reduce(A, other) with nothing recorded for backward.  `meanwhile` (optional): work of the caller that does
    not need the result; a row-sharded source runs it while its first exchange is in flight."""
    from .dist import ShardedSparseTensor
    if isinstance(src, ShardedSparseTensor):
        out = src.aggregate(other, reduce, meanwhile=meanwhile)
        if out is not None:
            return out
    if meanwhile is not None:
        meanwhile()
    operand = _operand(src, other, tag)
    if isinstance(src, ShardedSparseTensor):
        return ext_spmm._spmm(src.rowptr, src.col, src.value, operand, reduce)
    rowptr, col, value = src.csr()
    return ext_spmm._spmm(rowptr, col, value, operand, reduce)


def _aggregate_transposed(src, grad, reduce, rowscale=None, prescaled=False, tag="bw", meanwhile=None):
    """Gradient of reduce(A, other) with respect to `other` (spmm.cc:70-77, 128-137).  Inside the one-node
    layer the result is an fp32 regrouping of the separate nodes' anyway.
    With `rowscale` = 1 / max(deg, 1) the caller asks for A_mean^T g as A^T (D^-1 g): the rows of `grad` are
    scaled on the way into the SpMM and no per-edge weights are read (one load and one multiply per edge
    less: 10.0 against 12.0 ms at 125.8 M edges x 256 columns).  `prescaled`: `grad` already holds D^-1 g."""
    from .dist import ShardedSparseTensor
    if isinstance(src, ShardedSparseTensor):
        out = src.aggregate(grad, reduce, transposed=True, rowscale=rowscale, unweighted=prescaled, meanwhile=meanwhile)
        if out is not None:
            return out
    if meanwhile is not None:
        meanwhile()
    operand = _operand(src, grad, tag, rowscale)
    unweighted = rowscale is not None or prescaled
    if isinstance(src, ShardedSparseTensor):
        return ext_spmm._spmm(src.t_rowptr, src.t_col, None if unweighted else src.t_w, operand, "sum", regroup=True)
    t_ptr, t_col, t_w = src.storage.transposed("sum" if unweighted else reduce)
    return ext_spmm._spmm(t_ptr, t_col, None if unweighted else t_w, operand, "sum", regroup=True)


def _inverse_degree(src):
    """1 / max(deg, 1) of this rank's rows as an [rows] fp32 vector, or None when the adjacency carries
    edge values (the per-edge weights of the mean's transpose are then not a row scaling)."""
    from .dist import ShardedSparseTensor
    if isinstance(src, ShardedSparseTensor):
        if src.value is not None:
            return None
        inv = getattr(src, "_inv_deg", None)
        if inv is None:
            inv = (src.rowptr[1:] - src.rowptr[:-1]).to(torch.float32).clamp_(min=1).reciprocal_()
            src._inv_deg = inv
        return inv
    st = src.storage
    if st.value() is not None:
        return None
    inv = getattr(st, "_inv_deg", None)
    if inv is None:
        inv = st.rowcount().to(torch.float32).clamp_(min=1).reciprocal_()
        st._inv_deg = inv
    return inv


class qsage_layer(Function):
    """y = reduce(A, x) W_l^T + b (+ x W_r^T): the aggregation, lin_l and lin_r of QSAGEConv
    (layers.py:153-170) as one autograd node.  The compressed tensors saved are those of the separate
    nodes (x once, shared by the aggregation and lin_r; reduce(A, x) for lin_l) and are drawn in the same
    order.  What changes is the dense arithmetic around them:
      forward   one GEMM over the concatenated operands [reduce(A, x) | x] [W_l | W_r]^T + b;
      backward  grad_x = A^T (g W_l) + g W_r, with the transposed aggregation applied to g first when
                out_features < in_features ((A^T g) W_l: the SpMM, and the gradient all-gather of a
                row-sharded run, then work on out_features columns), and the second product accumulated
                into the first by the GEMM's epilogue.
    Results differ from the separate nodes by fp32 reassociation only."""

    @staticmethod
    @custom_fwd(device_type="cuda", cast_inputs=torch.float16)
    def forward(ctx, src, x, w_l, b_l, w_r, reduce, scheme_x, scheme_l):
        from .dist import ShardedSparseTensor
        # Row-sharded: what does not need the aggregate (compressing x, x W_r^T + b) is enqueued while the first
        # exchange of the aggregation is in flight; lin_l's product is then added to it.
        from .dist import column_split_active
        overlap = (isinstance(src, ShardedSparseTensor) and config.overlap_exchange
                   and column_split_active(src.world))
        early = {}

        def lin_r_early():
            if w_r is not None:
                early["y"] = ext_backward_func.linear_forward(x, w_r, b_l)

        def compress_x_and_lin_r():
            early["q"] = project_and_quantize(x, scheme_x, True)
            lin_r_early()

        out_f, in_f = w_l.shape
        k_agg = int(config.kept_frac * in_f + 0.999)
        kp, op = (k_agg + 3) // 4 * 4, (out_f + 3) // 4 * 4
        reorder = (config.aggregate_projected_first and config.kept_frac < 1.0 and config.compress_activation
                   and not config.simulate and not config.swap and x.dtype == torch.float32 and kp + op < in_f)
        if overlap and not reorder:
            agg = _aggregate(src, x, reduce, tag="fw%d" % x.size(1), meanwhile=compress_x_and_lin_r)
            q_x, randmat_x, proj_x = early["q"]
            if w_r is None:
                q_x = randmat_x = None
            q_agg, randmat_agg, proj_agg = project_and_quantize(agg, scheme_l, True)
            empty_cache(config.empty_cache_threshold)
            ctx.src, ctx.reduce = src, reduce
            ctx.saved = q_x, randmat_x, q_agg, randmat_agg, w_l, b_l, w_r
            ctx.other_args = x.shape, proj_x, proj_agg
            if w_r is None:
                return ext_backward_func.linear_forward(agg, w_l, b_l)
            return ext_backward_func.linear_forward(agg, w_l, None, out=early["y"], accumulate=True)
        # the input, compressed once (layers.py:153-159)
        q_x, randmat_x, proj_x = project_and_quantize(x, scheme_x, True)
        if w_r is None:
            q_x = randmat_x = None   # drawn (the noise stream stays that of the separate nodes), read by nothing
        if reorder:
            # Few outputs (the last layer): the aggregation is linear, so reduce(A, x) R = reduce(A, x R) and
            # reduce(A, x) W_l^T = reduce(A, x W_l^T).  One GEMM forms [x R | x W_l^T], the SpMM (and, row-
            # sharded, both exchanges) then works on k + out_features columns instead of in_features, and its
            # result holds the projected aggregate that lin_l saves (ops.py:142-149) and lin_l's output.  R and
            # the rounding noise are drawn where the separate nodes draw them.
            with torch.no_grad():
                off_r, off_n = config.next_offset(), config.next_offset()
                randmat_agg = _rademacher(in_f, k_agg, x.device, x.dtype, offset=off_r)
                wcat = x.new_zeros((kp + op, in_f))
                wcat[:k_agg].copy_(randmat_agg.t())
                wcat[kp:kp + out_f].copy_(w_l)
                t = _aggregate(src, ext_backward_func.linear_forward(x, wcat), reduce, tag="fw%d" % (kp + op),
                               meanwhile=lin_r_early if overlap else None)
                q_bits = config.activation_compression_bits[0]
                q_in, q_scale, q_min = ext_quantization.quantize_pack(t[:, :k_agg].contiguous(), q_bits, offset=off_n)
                q_agg = (q_in, q_bits, q_scale, q_min)
                if config.quantized_hook is not None:
                    config.quantized_hook(q_agg, randmat_agg)
                if "y" in early:
                    y = early["y"].add_(t[:, kp:kp + out_f])
                else:
                    y = t[:, kp:kp + out_f].contiguous()
                    if b_l is not None:
                        y += b_l
                    if w_r is not None:
                        y = ext_backward_func.linear_forward(x, w_r, None, out=y, accumulate=True)
            empty_cache(config.empty_cache_threshold)
            ctx.src, ctx.reduce = src, reduce
            ctx.saved = q_x, randmat_x, q_agg, randmat_agg, w_l, b_l, w_r
            ctx.other_args = x.shape, proj_x, torch.Size([x.shape[0], k_agg])
            return y
        agg = _aggregate(src, x, reduce, tag="fw%d" % x.size(1))
        q_agg, randmat_agg, proj_agg = project_and_quantize(agg, scheme_l, True)
        empty_cache(config.empty_cache_threshold)
        ctx.src, ctx.reduce = src, reduce
        ctx.saved = q_x, randmat_x, q_agg, randmat_agg, w_l, b_l, w_r
        ctx.other_args = x.shape, proj_x, proj_agg
        return ext_backward_func.linear_forward(agg, w_l, b_l, a2=x if w_r is not None else None, weight2=w_r)

    @staticmethod
    @custom_bwd(device_type="cuda")
    def backward(ctx, grad_output):
        q_x, randmat_x, q_agg, randmat_agg, w_l, b_l, w_r = ctx.saved
        x_shape, proj_x, proj_agg = ctx.other_args
        del ctx.saved
        g = grad_output.contiguous()
        k_agg, k_x = proj_agg[1], proj_x[1]
        both_projected = randmat_agg is not None and (w_r is None or randmat_x is not None)
        wg = {}
        pre = {}

        def bias_grad():
            # grad_output.sum(0) (backward_func.cc:88-90); already formed when the pass that scales g also summed it
            if "colsum" not in pre:
                pre["colsum"] = ext_backward_func.rows_scale_colsum(g)[1]
            return pre["colsum"]

        def weight_grads():
            grad_w_r = None
            if (config.compress_activation and not config.simulate and not config.swap and q_agg[1] is not None
                    and config.grad_weight_in_projected_space and both_projected
                    and ext_backward_func.grad_weight_supported(g, k_agg, k_x if w_r is not None else 0, q_agg[1])):
                # both weight gradients in one pass over g: g^T [Xq_agg | Xq_x] on the tensor cores, dequantised
                # on the way in, then the two small transposed projections
                ga, gx = ext_backward_func.grad_weight_from_packed(g, q_agg, k_agg, q_x if w_r is not None else None,
                                                                   k_x)
                grad_w_l = ga.mm(randmat_agg.t())
                grad_b = bias_grad() if b_l is not None else None
                if w_r is not None:
                    grad_w_r = gx.mm(randmat_x.t())
            else:
                _, grad_w_l, grad_b = linear_backward_from_compressed(q_agg, w_l, b_l, randmat_agg, x_shape, proj_agg,
                                                                      True, g, False)
                if w_r is not None:
                    _, grad_w_r, _ = linear_backward_from_compressed(q_x, w_r, None, randmat_x, x_shape, proj_x, True,
                                                                     g, False)
            wg["l"], wg["b"], wg["r"] = grad_w_l, grad_b, grad_w_r

        out_f, in_f = w_l.shape
        # row-sharded: the weight gradients are enqueued while the first exchange of the aggregation is in flight
        aggregated_first = ctx.needs_input_grad[1] and config.aggregate_gradient_first and out_f <= in_f
        if not aggregated_first:
            weight_grads()
        grad_x = None
        if ctx.needs_input_grad[1]:
            # With out_features <= in_features the transposed aggregation runs on g itself: fewer (or as
            # many) columns for the SpMM, one GEMM over [A^T g | g] instead of two, and, row-sharded, a
            # gathered operand that has passed the ReLU / dropout masks (mostly zeros, sent compacted)
            # instead of the dense g W_l.
            if config.aggregate_gradient_first and out_f <= in_f:
                pad = (-out_f) % 4   # whole 128-bit column groups for the gather
                inv = _inverse_degree(ctx.src) if ctx.reduce == "mean" else None
                gp, wp = g, w_l
                prescaled = False
                from .dist import ShardedSparseTensor
                if not isinstance(ctx.src, ShardedSparseTensor) and (inv is not None or pad):
                    # one pass over g: D^-1 g (zero-padded to whole column groups) and, for the bias, g.sum(0).
                    # (A row-sharded source scales the rows inside its exchange kernels instead.)
                    gp, colsum = ext_backward_func.rows_scale_colsum(g, inv, want_scaled=True,
                                                                     want_colsum=b_l is not None)
                    if colsum is not None:
                        pre["colsum"] = colsum
                    prescaled, inv = inv is not None, None
                    if pad:
                        wp = w_l.new_zeros((out_f + pad, in_f))
                        wp[:out_f].copy_(w_l)
                elif pad:
                    gp = g.new_zeros((g.size(0), out_f + pad))
                    if inv is not None:
                        torch.mul(g, inv.unsqueeze(1), out=gp[:, :out_f])   # pad and scale in one pass
                        inv, prescaled = None, True
                    else:
                        gp[:, :out_f].copy_(g)
                    wp = w_l.new_zeros((out_f + pad, in_f))
                    wp[:out_f].copy_(w_l)
                t = _aggregate_transposed(ctx.src, gp, ctx.reduce, rowscale=inv, prescaled=prescaled,
                                          tag="bw%d" % gp.size(1), meanwhile=weight_grads)
                grad_x = ext_backward_func.linear_forward(t, wp.t(), None, a2=g if w_r is not None else None,
                                                          weight2=w_r.t() if w_r is not None else None)
            else:
                grad_x = _aggregate_transposed(ctx.src, ext_backward_func.linear_forward(g, w_l.t()), ctx.reduce)
                if w_r is not None:
                    grad_x = ext_backward_func.linear_forward(g, w_r.t(), None, out=grad_x, accumulate=True)
        return None, grad_x, wg["l"], wg["b"], wg["r"], None, None, None


def sage_layer_applies(src):
    """Whether QSAGEConv runs as the one-node layer: no edge-value gradient, and the aggregation's own
    compressed copy (read only by the edge-value gradient) not being kept."""
    from .dist import ShardedSparseTensor
    if not (config.fuse_sage_layer and config.skip_dead_saves):
        return False
    if torch.is_autocast_enabled("cuda"):
        return False   # fp16 operands take the reference's three nodes (half arithmetic of its half kernels)
    if isinstance(src, ShardedSparseTensor):
        return True
    value = src.storage.value()
    return value is None or not value.requires_grad
