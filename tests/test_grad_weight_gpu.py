"""exact_grad_weight_from_packed (g^T . dequantise(packed) on the tensor cores) against the unpack -> fp64
product of the same packed activations: 2e-3 relative Frobenius (tf32 inputs), status word clear, one or two
activations, every bit width, ragged row counts, and inside the layers' backward."""
import numpy as np
import pytest
import torch

from exact_b200 import config
from exact_b200.cpp_extension import backward_func as B
from exact_b200.cpp_extension import quantization as Q

pytestmark = pytest.mark.gpu


def _packed(N, k, bits, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    x = torch.randn(N, k, device="cuda", generator=g)
    pk, sb, mb = Q.quantize_pack(x, bits, seed=seed, offset=0, row_offset=0)
    xh = Q.unpack_single_precision(pk, bits, sb, mb, N, k)
    return (pk, bits, sb, mb), xh


def rel(a, b):
    return float((a.double() - b.double()).norm() / (b.double().norm() + 1e-30))


@pytest.mark.parametrize("N,O,k0,k1,bits", [
    (20000, 256, 32, 32, 2), (20000, 256, 32, 0, 2), (4097, 128, 13, 32, 2), (50001, 256, 76, 32, 2),
    (9000, 48, 32, 32, 2), (20000, 256, 16, 16, 1), (20000, 64, 32, 16, 4), (6000, 256, 16, 8, 8),
    (300000, 256, 32, 32, 2), (4100, 100, 25, 0, 2),
])
def test_grad_weight_from_packed(N, O, k0, k1, bits):
    config.check_device_status = True
    config.grad_weight_tensor_core = True
    gen = torch.Generator(device="cuda").manual_seed(7)
    g = torch.randn(N, O, device="cuda", generator=gen)
    q0, x0 = _packed(N, k0, bits, 1)
    q1, x1 = _packed(N, k1, bits, 2) if k1 else (None, None)
    assert B.grad_weight_supported(g, k0, k1, bits)
    a, b = B.grad_weight_from_packed(g, q0, k0, q1, k1)
    ref_a = g.double().t() @ x0.double()
    assert a.shape == (O, k0) and rel(a, ref_a) < 2e-3
    if k1:
        ref_b = g.double().t() @ x1.double()
        assert b.shape == (O, k1) and rel(b, ref_b) < 2e-3
    # a second call gives the same bits (partials are added in a fixed order)
    a2, _ = B.grad_weight_from_packed(g, q0, k0, q1, k1)
    assert torch.equal(a, a2)
    config.check_device_status = False


def test_width_that_is_not_a_multiple_of_four_goes_in_padded():
    """47 classes: rows of 188 bytes cannot be described by a tensor map; g goes in as a zero-padded copy."""
    from exact_b200.cpp_extension import quantization as Q
    g = torch.randn(5000, 47, device="cuda")
    assert B.grad_weight_supported(g, 32, 32, 2)
    x = torch.randn(5000, 32, device="cuda")
    pk, sb, mb = Q.quantize_pack(x, 2, seed=3, offset=0)
    a, _ = B.grad_weight_from_packed(g, (pk, 2, sb, mb), 32)
    ref = g.t().double() @ Q.unpack_single_precision(pk, 2, sb, mb, 5000, 32).double()
    assert a.shape == (47, 32) and float((a.double() - ref).norm() / ref.norm()) < 2e-3


def test_unsupported_shapes_use_the_library_route():
    g = torch.randn(1000, 256, device="cuda")          # too few rows to be worth it
    assert not B.grad_weight_supported(g, 32, 32, 2)
    g = torch.randn(5000, 256, device="cuda")
    assert not B.grad_weight_supported(g, 256, 0, 2)   # more activation columns than the producers take
    config.grad_weight_tensor_core = False
    assert not B.grad_weight_supported(g, 32, 32, 2)
    config.grad_weight_tensor_core = True


def test_layer_backward_matches_the_unpack_route():
    """qlinear and the one-node GraphSAGE layer give the same gradients (2e-3) with the switch on and off."""
    from exact_b200 import QModule, graphs, models
    import torch.nn.functional as F
    dev = torch.device("cuda")
    adj = graphs.build_graph("cfg4", 0, dev, nodes=6000)
    adj.fill_cache_()
    adj.to_int32_()
    x = torch.randn(6000, 100, device=dev)
    y = torch.randint(47, (6000,), device=dev)
    grads = []
    for flag in (True, False):
        config.grad_weight_tensor_core = flag
        config.compress_activation, config.kept_frac, config.activation_compression_bits = True, 0.125, [2]
        config.manual_seed(3)
        torch.manual_seed(0)
        net = QModule(models.SAGE(100, 256, 47, 3, dropout=0.5)).to(dev).train()
        F.cross_entropy(net(x, adj), y).backward()
        grads.append({k: p.grad.clone() for k, p in net.named_parameters()})
    config.grad_weight_tensor_core = True
    config.kept_frac = 1.0
    for k in grads[0]:
        assert rel(grads[0][k], grads[1][k]) < 2e-3, k
