"""QModule: wraps a model and swaps its layers for the quantised ones (exact/exact/module.py:18-111),
for the layer types of the GCN / GraphSAGE path."""
from collections import OrderedDict

import torch.nn as nn

from . import _lib
from .conf import config
from .layers import (ActDropout, GCNConv, QBatchNorm1d, QDropout, QDropout2, QGCNConv, QLinear, QReLU,
                     QReLUDropout, QSAGEConv, SAGEConv)


class QModule(nn.Module):
    def __init__(self, model):
        super().__init__()
        self.model = model
        QModule.convert_layers(model)

    @staticmethod
    def convert_layers(module):
        """module.py:24-88."""
        for name, child in module.named_children():
            if isinstance(child, (QBatchNorm1d, QLinear, QReLU, QGCNConv, QDropout, QDropout2, QSAGEConv,
                                  QReLUDropout)):
                continue
            if (isinstance(child, ActDropout) and isinstance(child.activation, nn.ReLU)
                    and isinstance(child.dropout, nn.Dropout) and config.fuse_relu_dropout and not config.dropout2):
                setattr(module, name, QReLUDropout(child.dropout.p))
                continue
            if isinstance(child, nn.BatchNorm1d) and config.enable_quantized_bn:
                setattr(module, name, QBatchNorm1d(child.num_features, child.eps, child.momentum, child.affine,
                                                   child.track_running_stats))
            elif isinstance(child, nn.Linear):
                setattr(module, name, QLinear(child.in_features, child.out_features, child.bias is not None))
            elif isinstance(child, nn.ReLU):
                setattr(module, name, QReLU())
            elif isinstance(child, nn.Dropout):
                setattr(module, name, QDropout2(child.p) if config.dropout2 else QDropout(child.p))
            elif isinstance(child, GCNConv):
                setattr(module, name, QGCNConv(child.in_channels, child.out_channels, child.improved, child.cached,
                                               child.add_self_loops, child.normalize, child.bias is not None,
                                               aggr=child.aggr))
            elif isinstance(child, SAGEConv):
                setattr(module, name, QSAGEConv(child.in_channels, child.out_channels, child.normalize,
                                                child.root_weight, child.lin_l.bias is not None))
            else:
                QModule.convert_layers(child)

    def forward(self, *args, **kwargs):
        if self.training and config.poll_device_status:
            # one step late and without waiting for the GPU: raises if a kernel of an earlier step gave up on
            # a bounded on-chip wait (its outputs were incomplete)
            for a in args:
                if getattr(a, "is_cuda", False):
                    _lib.poll_status(a.device)
                    break
        return self.model(*args, **kwargs)

    def load_state_dict(self, state_dict, strict=True):
        """module.py:93-97: accept a checkpoint of the unwrapped model."""
        new_state_dict = OrderedDict([("model." + k, v) for k, v in state_dict.items()])
        return super().load_state_dict(new_state_dict, strict)

    def state_dict(self, destination=None, prefix="", keep_vars=False):
        """module.py:99-104: strip the wrapper's "model." prefix."""
        ret = super().state_dict(destination=destination, prefix=prefix, keep_vars=keep_vars)
        return OrderedDict([(k[6:], v) for k, v in ret.items()])

    def reset_parameters(self):
        self.model.reset_parameters()
