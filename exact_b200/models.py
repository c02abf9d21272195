"""The GCN and GraphSAGE model definitions the benchmarks train
(mem_speed_bench/models/gcn.py:11-64, mem_speed_bench/models/sage.py:13-77), written with the plain
layers of this package so that QModule can convert them."""
import torch
from torch.nn import BatchNorm1d, ModuleList

from .layers import ActDropout, GCNConv, SAGEConv


class GCN(torch.nn.Module):
    def __init__(self, in_channels, hidden_channels, out_channels, num_layers, dropout=0.0, drop_input=False,
                 batch_norm=False, residual=False):
        super().__init__()
        self.in_channels, self.out_channels = in_channels, out_channels
        self.dropout = torch.nn.Dropout(p=dropout)
        self.drop_input = drop_input
        if drop_input:
            self.input_dropout = torch.nn.Dropout(p=dropout)
        self.activation = torch.nn.ReLU()
        self.act_drop = ActDropout(self.activation, self.dropout)   # the pair applied after every hidden layer
        self.batch_norm, self.residual, self.num_layers = batch_norm, residual, num_layers
        self.convs = ModuleList()
        for i in range(num_layers):
            in_dim = in_channels if i == 0 else hidden_channels
            out_dim = out_channels if i == num_layers - 1 else hidden_channels
            self.convs.append(GCNConv(in_dim, out_dim, normalize=False))
        if self.batch_norm:
            self.bns = ModuleList(BatchNorm1d(hidden_channels) for _ in range(num_layers - 1))

    def reset_parameters(self):
        for conv in self.convs:
            conv.reset_parameters()
        if self.batch_norm:
            for bn in self.bns:
                bn.reset_parameters()

    def forward(self, x, adj_t, *args):
        if self.drop_input:
            x = self.input_dropout(x)
        for idx, conv in enumerate(self.convs[:-1]):
            h = conv(x, adj_t)
            if self.batch_norm:
                h = self.bns[idx](h)
            if self.residual and h.size(-1) == x.size(-1):
                h = h + x[:h.size(0)]
            x = self.act_drop(h)
        return self.convs[-1](x, adj_t)


class SAGE(torch.nn.Module):
    def __init__(self, in_channels, hidden_channels, out_channels, num_layers, dropout=0.0, batch_norm=False,
                 residual=False, use_linear=False):
        super().__init__()
        self.in_channels, self.out_channels = in_channels, out_channels
        self.dropout = torch.nn.Dropout(p=dropout)
        self.activation = torch.nn.ReLU()
        self.act_drop = ActDropout(self.activation, self.dropout)   # the pair applied after every hidden layer
        self.batch_norm, self.residual, self.num_layers = batch_norm, residual, num_layers
        self.use_linear = use_linear
        self.convs = ModuleList()
        if use_linear:
            self.lins = ModuleList()
        for i in range(num_layers):
            in_dim = in_channels if i == 0 else hidden_channels
            out_dim = out_channels if i == num_layers - 1 else hidden_channels
            self.convs.append(SAGEConv(in_dim, out_dim))
            if use_linear:
                self.lins.append(torch.nn.Linear(in_dim, out_dim, bias=False))
        if self.batch_norm:
            self.bns = ModuleList(BatchNorm1d(hidden_channels) for _ in range(num_layers - 1))

    def reset_parameters(self):
        for conv in self.convs:
            conv.reset_parameters()
        if self.batch_norm:
            for bn in self.bns:
                bn.reset_parameters()
        if self.use_linear:
            for lin in self.lins:
                lin.reset_parameters()

    def forward(self, x, adj_t, *args):
        for idx, conv in enumerate(self.convs[:-1]):
            h = conv(x, adj_t)
            if self.use_linear:
                h = h + self.lins[idx](x)
            if self.batch_norm:
                h = self.bns[idx](h)
            if self.residual and h.size(-1) == x.size(-1):
                h = h + x[:h.size(0)]
            x = self.act_drop(h)
        h = self.convs[-1](x, adj_t)
        if self.use_linear:
            h = h + self.lins[-1](x)
        return h
