"""CPU restatement of the reference's layer wiring for GCN / GraphSAGE -- TEST INFRASTRUCTURE ONLY.

torch (CPU) autograd Functions whose compressed-activation arithmetic runs through the C oracle; the
dense GEMMs and batch norm are torch CPU calls, as they are ATen calls in the reference.  Follows
exact/exact/ops.py:128-178 (qlinear), 206-254 (qbatch_norm), 257-371 (qspmm_sum / qspmm_mean),
exact/exact/layers.py:142-174 (QSAGEConv), 226-262 (QGCNConv) and the model definitions in
mem_speed_bench/models/{gcn,sage}.py.  Noise is the B200 library's Philox stream restated in the
oracle, drawn in the same call order as exact_b200 draws it, so that a GPU run and this CPU run of the
same model see the same stochastic rounding, dropout masks and projection matrices.

Used by the parity tests of the layer stack and as the timed CPU baseline of the benchmark."""
import numpy as np
import torch
import torch.nn.functional as F

import oracle


class Noise:
    """(seed, running offset): the counterpart of exact_b200.config.seed / next_offset()."""

    def __init__(self, seed=0):
        self.seed = int(seed)
        self.offset = 0

    def next(self):
        o = self.offset
        self.offset += 1
        return o


class Cfg:
    def __init__(self, bits=2, kept_frac=1.0, compress=True, seed=0, fused_rp=False):
        self.bits, self.kept_frac, self.compress = bits, kept_frac, compress
        self.noise = Noise(seed)
        # the B200 library's fused projection+pack kernel keys its noise by (row, block of 8 columns)
        self.fused_rp = fused_rp


def _rp_fused(cfg, D, k):
    # the shapes the fused kernel takes: any D, k up to 512 with three pipeline stages in shared memory
    kpad = (k + 15) // 16 * 16
    return cfg.fused_rp and kpad <= 512 and 200 * 1024 // (128 * 128 + kpad * 128) >= (3 if D % 4 else 2)


def _np(t):
    return t.detach().contiguous().numpy()


def compress(cfg, x, rp=True, fused=None):
    """(input2rp ->) quantize_activation: exact/exact/ops.py:142-149 -> saved tuple.  `fused` = False: the CUDA
    side quantises this tensor with the plain pack kernel (its noise stream) whatever the shape."""
    x = _np(x)
    N, D = x.shape
    R = None
    rows_keyed = False
    if cfg.kept_frac < 1.0 and rp:
        k = int(cfg.kept_frac * D + 0.999)
        R = oracle.rademacher(cfg.noise.seed, cfg.noise.next(), D, k)
        x = oracle.input2rp(x, R)
        rows_keyed = _rp_fused(cfg, D, k) and cfg.compress and fused is not False
    if not cfg.compress:
        return ("raw", x.copy(), R, (N, D))
    if rows_keyed:
        u = oracle.noise_b200_rows(cfg.noise.seed, cfg.noise.next(), x.shape[0], x.shape[1])
    else:
        u = oracle.noise_b200(cfg.noise.seed, cfg.noise.next(), x.shape[0], x.shape[1])
    packed, sb, mb, _, _ = oracle.quantize_activation(x, u, cfg.bits)
    return ("q", (packed, sb, mb, x.shape), R, (N, D))


def decompress(cfg, saved):
    """dequantize_activation (-> rp2input): ops.py:164-166."""
    kind, payload, R, shape = saved
    if kind == "raw":
        x = payload
    else:
        packed, sb, mb, pshape = payload
        x = oracle.dequantize_activation(packed, sb, mb, pshape[0], pshape[1], cfg.bits)
    if R is not None:
        x = oracle.rp2input(x, R)
    return torch.from_numpy(x.reshape(shape))


class OQLinear(torch.autograd.Function):
    """ops.py:128-178."""

    @staticmethod
    def forward(ctx, cfg, x, weight, bias, saved):
        ctx.cfg = cfg
        ctx.saved_act = compress(cfg, x) if saved is None else saved
        ctx.save_for_backward(weight)
        ctx.has_bias = bias is not None
        return F.linear(x, weight, bias)

    @staticmethod
    def backward(ctx, g):
        (weight,) = ctx.saved_tensors
        xh = decompress(ctx.cfg, ctx.saved_act)
        gi = g.mm(weight)                 # backward_func.cc:86-91
        gw = g.t().mm(xh)
        gb = g.sum(0) if ctx.has_bias else None
        return None, gi, gw, gb, None


class OSpmm(torch.autograd.Function):
    """ops.py:257-371; gradient with respect to the dense operand only (spmm.cc:70-77, 128-137)."""

    @staticmethod
    def forward(ctx, adj, x, reduce):
        ctx.adj, ctx.reduce = adj, reduce
        rowptr, col, val = adj
        return torch.from_numpy(oracle.spmm(rowptr, col, val, _np(x), reduce))

    @staticmethod
    def backward(ctx, g):
        rowptr, col, val = ctx.adj
        n_cols = rowptr.size - 1
        return None, torch.from_numpy(oracle.spmm_bw_mat(rowptr, col, val, _np(g), n_cols, ctx.reduce)), None


class OReLU(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        out, keep = oracle.relu_fw(_np(x))
        ctx.keep = keep
        return torch.from_numpy(out)

    @staticmethod
    def backward(ctx, g):
        return torch.from_numpy(oracle.mask_bw(_np(g), ctx.keep))


class ODropout(torch.autograd.Function):
    @staticmethod
    def forward(ctx, cfg, x, p):
        xn = _np(x)
        u = oracle.uniform_b200(cfg.noise.seed, cfg.noise.next(), xn.size).reshape(xn.shape)
        out, keep = oracle.dropout_fw(xn, u, p)
        ctx.keep, ctx.p = keep, p
        return torch.from_numpy(out)

    @staticmethod
    def backward(ctx, g):
        return None, torch.from_numpy(oracle.dropout_bw(_np(g), ctx.keep, ctx.p)), None


class OBatchNorm(torch.autograd.Function):
    """ops.py:206-254: input saved compressed (never projected), ATen batch norm forward/backward."""

    @staticmethod
    def forward(ctx, cfg, x, weight, bias, eps):
        ctx.cfg, ctx.eps = cfg, eps
        ctx.saved_act = compress(cfg, x, rp=False)
        out, mean, invstd = torch.ops.aten.native_batch_norm(x, weight, bias, None, None, True, 0.1, eps)
        ctx.save_for_backward(weight, mean, invstd)
        return out

    @staticmethod
    def backward(ctx, g):
        weight, mean, invstd = ctx.saved_tensors
        xh = decompress(ctx.cfg, ctx.saved_act)
        gi, gw, gb = torch.ops.aten.native_batch_norm_backward(g.contiguous(), xh, weight, None, None, mean, invstd,
                                                               True, ctx.eps, [True, True, True])
        return None, gi, gw, gb, None


def gcn_forward(cfg, params, x, adj, n_layers, batch_norm, dropout):
    """mem_speed_bench/models/gcn.py:51-64 with QGCNConv (layers.py:226-262): qlinear (no bias), SpMM
    sum with the normalised values, + bias; BN, ReLU, dropout between layers."""
    for i in range(n_layers):
        h = OQLinear.apply(cfg, x, params[f"convs.{i}.weight"], None, None)
        h = OSpmm.apply(adj, h, "sum")
        h = h + params[f"convs.{i}.bias"]
        if i == n_layers - 1:
            return h
        if batch_norm:
            h = OBatchNorm.apply(cfg, h, params[f"bns.{i}.weight"], params[f"bns.{i}.bias"], 1e-5)
        x = OReLU.apply(h)
        x = ODropout.apply(cfg, x, dropout)   # the models always call their Dropout module, p = 0 included


def sage_forward(cfg, params, x, adj, n_layers, dropout):
    """mem_speed_bench/models/sage.py:59-77 with QSAGEConv (layers.py:142-174): one compressed copy of
    the input shared by the mean aggregation and lin_r; lin_l compresses the aggregate."""
    for i in range(n_layers):
        shared = compress(cfg, x)
        agg = OSpmm.apply(adj, x, "mean")
        # The CUDA layer with few outputs aggregates [x R | x W_l^T] (the same numbers up to fp32 reassociation) and
        # then packs the projected aggregate with the plain pack kernel: same values, that kernel's noise stream.
        w_l = params[f"convs.{i}.lin_l.weight"]
        k = int(cfg.kept_frac * w_l.shape[1] + 0.999)
        pad4 = lambda v: (v + 3) // 4 * 4
        reordered = (getattr(cfg, "reorder_sage", True) and cfg.kept_frac < 1.0 and cfg.compress
                     and pad4(k) + pad4(w_l.shape[0]) < w_l.shape[1])
        saved_agg = compress(cfg, agg, fused=False) if reordered else None
        h = OQLinear.apply(cfg, agg, w_l, params[f"convs.{i}.lin_l.bias"], saved_agg)
        h = h + OQLinear.apply(cfg, x, params[f"convs.{i}.lin_r.weight"], None, shared)
        if i == n_layers - 1:
            return h
        x = OReLU.apply(h)
        x = ODropout.apply(cfg, x, dropout)   # the models always call their Dropout module, p = 0 included


def train_step(cfg, model, params, x, adj, y, n_layers, batch_norm=False, dropout=0.0):
    """One full-batch step: forward, cross-entropy over all nodes, backward.  -> (loss, grads dict)."""
    params = {k: v.detach().clone().requires_grad_() for k, v in params.items()}
    if model == "gcn":
        out = gcn_forward(cfg, params, x, adj, n_layers, batch_norm, dropout)
    else:
        out = sage_forward(cfg, params, x, adj, n_layers, dropout)
    loss = F.cross_entropy(out, y)
    loss.backward()
    return loss.item(), out.detach(), {k: v.grad for k, v in params.items()}
