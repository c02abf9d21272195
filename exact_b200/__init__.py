"""exact_b200: the activation-compression hot path of EXACT (zirui-ray-liu/Exact) on NVIDIA B200.

The public names are those of the reference's `exact` package (exact/exact/__init__.py:1-5) for the
GCN / GraphSAGE path.  All arithmetic of the path runs in libexact_b200.so (hand-written sm_100a CUDA,
C ABI in include/exact_b200.h); there is no CPU or eager fallback."""
from .conf import config
from .utils import cast_low_bit_int, compute_tensor_bytes, get_memory_usage
from .sparse import SparseTensor, gcn_norm
from .ops import (dequantize_activation, input2rp, qbatch_norm, qlinear, qspmm_mean, qspmm_sum,
                  quantize_activation, rp2input)
from .spmm import QMatmul, qmatmul
from .layers import (GCNConv, QBatchNorm1d, QDropout, QDropout2, QGCNConv, QLeakyReLU, QLinear, QReLU, QSAGEConv,
                     SAGEConv)
from .module import QModule
from ._lib import ExactB200Error, check_status, poll_status

__all__ = [
    "config", "QModule", "QGCNConv", "QSAGEConv", "QLinear", "QReLU", "QLeakyReLU", "QDropout", "QDropout2", "QBatchNorm1d",
    "QMatmul", "qmatmul", "GCNConv", "SAGEConv", "SparseTensor", "gcn_norm", "quantize_activation",
    "dequantize_activation", "input2rp", "rp2input", "qlinear", "qbatch_norm", "qspmm_sum", "qspmm_mean",
    "ExactB200Error", "check_status", "poll_status", "get_memory_usage", "compute_tensor_bytes", "cast_low_bit_int",
]
