"""QScheme: the per-layer quantisation scheme object of the reference (exact/exact/qsheme.py:8-48).
Only the live part is kept: layer naming/counters and compute_quantization_bits, which yields the
same row min/max as the scheme-less path (ops.py:61-66).  The unused calc_precision import is dropped."""
import torch

from .conf import config


class QScheme(object):
    num_samples = 1
    num_matmul_layer = 0
    num_lin_layer = 0
    num_batchnorm_layer = 0
    num_sage_layer = 0
    batch = None
    update_scale = True
    layers = []
    prev_layer = None

    def __init__(self, name):
        self.initial_bits = config.initial_bits
        self.bits = config.activation_compression_bits[0]
        QScheme.layers.append(self)
        assert name in ["linear", "matmul", "batchnorm", "sage"]
        counter = {"linear": "num_lin_layer", "matmul": "num_matmul_layer",
                   "batchnorm": "num_batchnorm_layer", "sage": "num_sage_layer"}[name]
        self.name = f"{name}_{getattr(QScheme, counter)}"
        setattr(QScheme, counter, getattr(QScheme, counter) + 1)

    def compute_quantization_bits(self, input):
        """qsheme.py:41-48 -> (input [N, -1], bits, row min, row max)."""
        QScheme.prev_layer = self
        N = input.shape[0]
        input_flatten = input.view(N, -1)
        mn, mx = torch.min(input_flatten, 1)[0], torch.max(input_flatten, 1)[0]
        b = config.activation_compression_bits[0]
        return input_flatten, b, mn, mx
