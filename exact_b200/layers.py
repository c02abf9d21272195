"""Quantised nn.Modules with the reference's names and constructor arguments
(exact/exact/layers.py).  torch_geometric is not a dependency: GCNConv and SAGEConv below restate the
parts of PyG 1.7.2's layers that the reference's subclasses and QModule rely on (attributes read at
module.py:41-56, parameter shapes, initialisation, forward on a SparseTensor adjacency)."""
import math

import torch
import torch.nn.functional as F
from torch import Tensor
from torch.nn import Parameter

from .conf import config
from .cpp_extension import quantization as ext_quantization
from .ops import project_and_quantize, qbatch_norm, qlinear
from .qscheme import QScheme
from .sparse import SparseTensor, gcn_norm
from .spmm import QMatmul, qmatmul, qsage_layer, sage_layer_applies


def _glorot(t):
    if t is not None:
        stdv = math.sqrt(6.0 / (t.size(-2) + t.size(-1)))
        t.data.uniform_(-stdv, stdv)


# ----------------------------------------------------------------------------------------------------
# Plain (uncompressed) layers: what a model is written with before QModule converts it.
class GCNConv(torch.nn.Module):
    """torch_geometric.nn.GCNConv (1.7.2) on a SparseTensor adjacency: out = A_hat (x W) + b."""

    def __init__(self, in_channels, out_channels, improved=False, cached=False, add_self_loops=True,
                 normalize=True, bias=True, aggr="add"):
        super().__init__()
        self.in_channels, self.out_channels = in_channels, out_channels
        self.improved, self.cached = improved, cached
        self.add_self_loops, self.normalize, self.aggr = add_self_loops, normalize, aggr
        self._cached_adj_t = None
        self.weight = Parameter(torch.empty(in_channels, out_channels))
        if bias:
            self.bias = Parameter(torch.empty(out_channels))
        else:
            self.register_parameter("bias", None)
        self.reset_parameters()

    def reset_parameters(self):
        _glorot(self.weight)
        if self.bias is not None:
            self.bias.data.zero_()
        self._cached_adj_t = None

    def _norm(self, adj_t):
        if not self.normalize:
            return adj_t
        if self._cached_adj_t is not None:
            return self._cached_adj_t
        out = gcn_norm(adj_t, add_self_loops=self.add_self_loops)
        if self.cached:
            self._cached_adj_t = out
        return out

    def forward(self, x, adj_t, edge_weight=None):
        adj_t = self._norm(adj_t)
        x = x @ self.weight
        out = qmatmul_plain(adj_t, x, "sum")
        if self.bias is not None:
            out = out + self.bias
        return out


class SAGEConv(torch.nn.Module):
    """torch_geometric.nn.SAGEConv (1.7.2), mean aggregation: out = W_l mean_j(x_j) + W_r x."""

    def __init__(self, in_channels, out_channels, normalize=False, root_weight=True, bias=True):
        super().__init__()
        self.in_channels, self.out_channels = in_channels, out_channels
        self.normalize, self.root_weight = normalize, root_weight
        self.aggr = "mean"
        if isinstance(in_channels, int):
            in_channels = (in_channels, in_channels)
        self.lin_l = torch.nn.Linear(in_channels[0], out_channels, bias=bias)
        if root_weight:
            self.lin_r = torch.nn.Linear(in_channels[1], out_channels, bias=False)
        self.reset_parameters()

    def reset_parameters(self):
        self.lin_l.reset_parameters()
        if self.root_weight:
            self.lin_r.reset_parameters()

    def forward(self, x, adj_t, size=None):
        if isinstance(x, Tensor):
            x = (x, x)
        out = qmatmul_plain(adj_t, x[0], "mean")
        out = self.lin_l(out)
        if self.root_weight and x[1] is not None:
            out = out + self.lin_r(x[1])
        if self.normalize:
            out = F.normalize(out, p=2.0, dim=-1)
        return out


def qmatmul_plain(adj_t, x, reduce):
    """Aggregation of the unconverted layers: the same SpMM kernel, nothing saved compressed."""
    saved = config.compress_activation, config.kept_frac
    config.compress_activation, config.kept_frac = False, 1.0
    try:
        return qmatmul(adj_t, x, reduce)
    finally:
        config.compress_activation, config.kept_frac = saved


# ----------------------------------------------------------------------------------------------------
class QLinear(torch.nn.Linear):
    """layers.py:268-281."""

    def __init__(self, input_features, output_features, bias=True, rp=True):
        super().__init__(input_features, output_features, bias)
        self.scheme = QScheme("linear") if config.single_precision else None
        self.rp = rp

    def forward(self, input, quantized=None, randmat=None):
        if self.training:
            return qlinear.apply(input, self.weight, self.bias, quantized, randmat, self.scheme, self.rp)
        return super().forward(input)


class QReLU(torch.nn.Module):
    """layers.py:284-292."""

    def __init__(self, inplace=False):
        super().__init__()

    def forward(self, input):
        if self.training:
            return ext_quantization.act_quantized_relu(input.contiguous())
        return F.relu(input)


class QLeakyReLU(torch.nn.Module):
    """layers.py:295-301 (the reference applies the masked kernel in training and in evaluation alike)."""

    def __init__(self, negative_slope, inplace=False):
        super().__init__()
        self.negative_slope = negative_slope

    def forward(self, input):
        return ext_quantization.act_quantized_leaky_relu(input, self.negative_slope)


class QDropout(torch.nn.Module):
    """layers.py:316-325."""

    def __init__(self, p):
        self.p = p
        super().__init__()

    def forward(self, input):
        if self.training:
            return ext_quantization.act_quantized_dropout(input.contiguous(), self.p, self.training)
        return F.dropout(input, self.p, self.training)


class ActDropout(torch.nn.Module):
    """activation followed by dropout, as the GCN / GraphSAGE models apply them after every hidden layer
    (mem_speed_bench/models/gcn.py:60-61, sage.py:72-73).  Kept as one child so that QModule can swap the
    pair for the one-pass QReLUDropout; unconverted it just calls the two modules."""

    def __init__(self, activation, dropout):
        super().__init__()
        self.activation, self.dropout = activation, dropout

    def forward(self, input):
        return self.dropout(self.activation(input))


class QReLUDropout(torch.nn.Module):
    """QReLU followed by QDropout (layers.py:284-292, 316-325) in one pass over the activation and with one
    saved 1-bit mask; outputs and gradients are those of the two modules."""

    def __init__(self, p):
        super().__init__()
        self.p = p

    def forward(self, input):
        if self.training:
            return ext_quantization.act_quantized_relu_dropout(input, self.p, True)
        return F.relu(input)


class QDropout2(torch.nn.Module):
    """layers.py:328-337."""

    def __init__(self, p):
        self.p = p
        super().__init__()

    def forward(self, input):
        if self.training:
            return ext_quantization.act_quantized_dropout(input.contiguous(), self.p, self.training) * (1 - self.p)
        return F.dropout(input, self.p, self.training) * (1 - self.p)


class QBatchNorm1d(torch.nn.BatchNorm1d):
    """layers.py:340-388."""

    def __init__(self, num_features, eps=1e-05, momentum=0.1, affine=True, track_running_stats=True):
        super().__init__(num_features, eps, momentum, affine, track_running_stats)
        self.scheme = QScheme("batchnorm") if config.single_precision else None

    def forward(self, input):
        if not self.training:
            return super().forward(input)
        self._check_input_dim(input)
        exponential_average_factor = 0.0 if self.momentum is None else self.momentum
        if self.training and self.track_running_stats and self.num_batches_tracked is not None:
            self.num_batches_tracked = self.num_batches_tracked + 1
            if self.momentum is None:
                exponential_average_factor = 1.0 / float(self.num_batches_tracked)
            else:
                exponential_average_factor = self.momentum
        bn_training = True
        return qbatch_norm.apply(
            input,
            self.running_mean if not self.training or self.track_running_stats else None,
            self.running_var if not self.training or self.track_running_stats else None,
            self.weight, self.bias, bn_training, exponential_average_factor, self.eps, self.scheme)


class QGCNConv(GCNConv):
    """layers.py:215-265.  The weight is [out_channels, in_channels] (layers.py:218), i.e. transposed
    with respect to the plain GCNConv."""

    def __init__(self, *args, **kwargs):
        super().__init__(*args, **kwargs)
        self.weight = Parameter(torch.empty(self.out_channels, self.in_channels))
        self.msg_and_aggr_func = QMatmul(self.aggr)
        self.lin_scheme = QScheme("linear") if config.single_precision else None
        self.reset_parameters()

    def forward(self, x, edge_index, edge_weight=None):
        adj_t = self._norm(edge_index)
        if self.training:
            # layers.py:252 passes lin_scheme in the `randmat` slot; the call is equivalent to this one.
            x = qlinear.apply(x, self.weight, None, None, None, self.lin_scheme, True)
        else:
            x = F.linear(x, self.weight, None)
        out = self.message_and_aggregate(adj_t, x)
        if self.bias is not None:
            out = out + self.bias
        return out

    def message_and_aggregate(self, adj_t, x):
        return self.msg_and_aggr_func(adj_t, x)


class QSAGEConv(SAGEConv):
    """layers.py:123-178: the input is projected and quantised once and that one compressed copy is
    shared by the aggregation and by lin_r."""

    def __init__(self, *args, **kwargs):
        super().__init__(*args, **kwargs)
        in_channels = self.in_channels
        if isinstance(in_channels, int):
            in_channels = (in_channels, in_channels)
        bias = self.lin_l.bias is not None
        self.lin_l = QLinear(in_channels[0], self.out_channels, bias=bias, rp=True)
        if self.root_weight:
            self.lin_r = QLinear(in_channels[1], self.out_channels, bias=False, rp=True)
        self.msg_and_aggr_func = QMatmul(self.aggr)
        self.scheme = QScheme("sage") if config.single_precision else None
        self.reset_parameters()

    def forward(self, x, edge_index, size=None):
        if isinstance(x, Tensor):
            x = (x, x)
            l_eq_r = True
        else:
            l_eq_r = False
        if l_eq_r and self.training and not self.normalize and sage_layer_applies(edge_index):
            return qsage_layer.apply(edge_index, x[0], self.lin_l.weight, self.lin_l.bias,
                                     self.lin_r.weight if self.root_weight else None,
                                     self.msg_and_aggr_func.reduce, self.scheme, self.lin_l.scheme)
        if l_eq_r and self.training:
            quantized, randmat, _ = project_and_quantize(x[0], self.scheme, True)
        else:
            quantized, randmat = None, None
        out = self.message_and_aggregate(edge_index, x, quantized=quantized, randmat=randmat)
        out = self.lin_l(out)
        x_r = x[1]
        if self.root_weight and x_r is not None:
            out = out + self.lin_r(x_r, quantized, randmat)
        if self.normalize:
            out = F.normalize(out, p=2.0, dim=-1)
        return out

    def message_and_aggregate(self, adj_t, x, quantized=None, randmat=None):
        return self.msg_and_aggr_func(adj_t, x[0], quantized=quantized, randmat=randmat)
