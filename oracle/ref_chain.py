"""The reference's own op chain for one quantised GraphSAGE training step, on the GPU, built from the
reference's UNMODIFIED CUDA kernels (oracle/_ref/ref_quantization.so, ref_spmm.so; see build_ref.py) and the
library calls the reference makes.  Checker / baseline side only: tests and the reference arm of bench.py
import it, the product never does.

It follows the reference's Python wiring call by call:
  quantize_activation   exact/exact/ops.py:61-83    torch.min / torch.max, scale = (2^b - 1) / (max - min),
                                                    pack_single_precision, statistics kept as bf16
  dequantize_activation ops.py:86-98                bf16 -> fp32, unpack_single_precision
  input2rp / rp2input   ops.py:107-125              randint signs / sqrt(k), torch.matmul
  qlinear               ops.py:128-178              F.linear forward; backward unpack -> rp2input ->
                                                    linear_backward (backward_func.cc:83-93: two mm + sum)
  qspmm_mean            ops.py:310-371              spmm_mean_fw / spmm_mean_bw (spmm.cc:84-139)
  QSAGEConv             layers.py:142-174           x compressed once, shared by the aggregation and lin_r
  model                 mem_speed_bench/models/sage.py:59-77   conv -> ReLU -> dropout ... conv
ReLU and dropout are torch's (F.relu, F.dropout): the reference's 1-bit-mask kernels store 16 mask words per
block regardless of the mask's length (quantization_cuda_kernel.cu:265-267), an out-of-bounds write for these
sizes, so they are not run."""
import math
import os
import sys

import torch
import torch.nn.functional as F

REF = os.path.join(os.path.dirname(os.path.abspath(__file__)), "_ref")


def available():
    return (torch.cuda.is_available() and os.path.exists(os.path.join(REF, "ref_quantization.so"))
            and os.path.exists(os.path.join(REF, "ref_spmm.so")))


def _mods():
    if REF not in sys.path:
        sys.path.insert(0, REF)
    import ref_quantization
    import ref_spmm
    return ref_quantization, ref_spmm


class Graph:
    """The index tensors QMatmul materialises for the mean aggregation (exact/exact/spmm.py:36-44)."""

    def __init__(self, rowptr, col):
        self.rowptr, self.col = rowptr.to(torch.int64), col.to(torch.int64)
        n = self.rowptr.numel() - 1
        self.rowcount = self.rowptr[1:] - self.rowptr[:-1]
        self.row = torch.repeat_interleave(torch.arange(n, device=col.device), self.rowcount)
        key = self.col * n + self.row
        self.csr2csc = torch.argsort(key)
        del key
        colcount = torch.bincount(self.col, minlength=n)
        self.colptr = torch.zeros(n + 1, dtype=torch.int64, device=col.device)
        torch.cumsum(colcount, 0, out=self.colptr[1:])


def quantize_activation(x, bits):
    rq, _ = _mods()
    mn, mx = torch.min(x, 1)[0], torch.max(x, 1)[0]
    scale = (2 ** bits - 1) / (mx - mn)
    packed = rq.pack_single_precision(x, mn, mx, scale, bits, True)
    return packed, bits, scale.to(torch.bfloat16), mn.to(torch.bfloat16)


def dequantize_activation(q, shape):
    rq, _ = _mods()
    packed, bits, scale, mn = q
    return rq.unpack_single_precision(packed, bits, scale.to(torch.float32), mn.to(torch.float32), shape[0],
                                      shape[1]).contiguous()


@torch.no_grad()
def input2rp(x, k):
    r = (2.0 * torch.randint(2, size=(x.shape[1], k), device=x.device) - 1.0) / math.sqrt(k)
    r = r.to(x.dtype)
    return torch.matmul(x, r), r


class QLinear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, b, quantized, randmat, cfg):
        if quantized is None:
            k = int(cfg["kept_frac"] * x.shape[1] + 0.999)
            xr, randmat = input2rp(x, k)
            quantized = quantize_activation(xr, cfg["bits"])
            del xr
        ctx.saved = quantized, w, b, randmat, x.shape
        return F.linear(x, w, b)

    @staticmethod
    def backward(ctx, g):
        quantized, w, b, randmat, shape = ctx.saved
        del ctx.saved
        xq = dequantize_activation(quantized, (shape[0], randmat.shape[1]))
        xh = torch.matmul(xq, randmat.t())
        del xq
        g = g.contiguous()
        grad_in = g.mm(w) if ctx.needs_input_grad[0] else None
        grad_w = g.t().mm(xh)
        grad_b = g.sum(0) if b is not None else None
        return grad_in, grad_w, grad_b, None, None, None


class SpmmMean(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, graph):
        _, rs = _mods()
        ctx.graph = graph
        g = graph
        return rs.spmm_mean_fw(g.row, g.rowptr, g.col, None, g.rowcount, g.colptr, g.csr2csc, x)

    @staticmethod
    def backward(ctx, grad_out):
        _, rs = _mods()
        g = ctx.graph
        dummy = torch.tensor([1.0], device=grad_out.device)
        _, grad_mat = rs.spmm_mean_bw(g.row, g.rowptr, g.col, g.col, g.rowcount, g.colptr, g.csr2csc, dummy,
                                      grad_out.contiguous(), False, False, True)
        return grad_mat, None


def sage_conv(x, graph, w_l, b_l, w_r, cfg):
    """layers.py:153-170."""
    k = int(cfg["kept_frac"] * x.shape[1] + 0.999)
    xr, randmat = input2rp(x, k)
    quantized = quantize_activation(xr, cfg["bits"])
    del xr
    out = SpmmMean.apply(x, graph)
    out = QLinear.apply(out, w_l, b_l, None, None, cfg)
    return out + QLinear.apply(x, w_r, None, quantized, randmat, cfg)


def sage_forward(params, x, graph, layers, dropout, cfg):
    """mem_speed_bench/models/sage.py:59-77 (batch_norm off)."""
    for i in range(layers):
        x = sage_conv(x, graph, params[f"convs.{i}.lin_l.weight"], params[f"convs.{i}.lin_l.bias"],
                      params[f"convs.{i}.lin_r.weight"], cfg)
        if i < layers - 1:
            x = F.relu(x)
            x = F.dropout(x, p=dropout, training=True)
    return x
