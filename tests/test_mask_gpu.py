"""GPU parity of the 1-bit-mask ReLU and dropout against torch and the CPU oracle."""
import numpy as np
import pytest
import torch
import torch.nn.functional as F

import oracle
from exact_b200.cpp_extension import quantization as Q
from helpers import normal, uniform01

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("shape", [(10000, 128), (169343, 3), (7,), (129, 5), (1, 1)])
def test_relu_equals_torch_relu(shape):
    # test/test_op.py:22-41
    x = np.random.default_rng(1).standard_normal(shape).astype(np.float32)
    a = torch.from_numpy(x).cuda().requires_grad_()
    b = torch.from_numpy(x).cuda().requires_grad_()
    go = torch.from_numpy(np.random.default_rng(2).standard_normal(shape).astype(np.float32)).cuda()
    ya, yb = F.relu(a), Q.act_quantized_relu(b)
    ya.backward(go)
    yb.backward(go)
    assert torch.equal(ya, yb) and torch.equal(a.grad, b.grad)
    out, keep = oracle.relu_fw(x)
    assert np.array_equal(yb.detach().cpu().numpy(), out)


def test_relu_unaligned_view():
    base = torch.randn(1000 * 128 + 1, device="cuda")
    x = base[1:].view(1000, 128).requires_grad_()   # 4-byte aligned only
    y = Q.act_quantized_relu(x)
    y.backward(torch.ones_like(y))
    assert torch.equal(y, F.relu(x.detach())) and torch.equal(x.grad, (x.detach() > 0).float())


@pytest.mark.parametrize("p", [0.5, 0.2, 0.75])
@pytest.mark.parametrize("shape", [(2330, 602), (1001, 7), (5,)])
def test_dropout_supplied_uniforms(shape, p):
    x = np.random.default_rng(3).standard_normal(shape).astype(np.float32)
    u = uniform01(shape, 4)
    g = np.random.default_rng(5).standard_normal(shape).astype(np.float32)
    xt = torch.from_numpy(x).cuda().requires_grad_()
    y = Q.act_quantized_dropout(xt, p, True, uniforms=torch.from_numpy(u).cuda())
    y.backward(torch.from_numpy(g).cuda())
    out, keep = oracle.dropout_fw(x, u, p)
    assert np.array_equal(y.detach().cpu().numpy(), out)
    assert np.array_equal(xt.grad.cpu().numpy(), oracle.dropout_bw(g, keep, p))


def test_dropout_philox_and_reference_test():
    # test/test_op.py:463-480 on the same all-ones 232,965 x 602 input
    x = torch.ones(232965, 602, device="cuda", requires_grad=True)
    from exact_b200 import config
    config.manual_seed(123)
    y = Q.act_quantized_dropout(x, 0.5, True)
    y.backward(torch.ones_like(y))
    assert torch.equal(y == 0, x.grad == 0)
    assert y.max().item() == 2.0 and x.grad.max().item() == 2.0
    assert abs((y != 0).float().mean().item() - 0.5) < 1e-3
    # the kernel's Philox stream equals the oracle's restatement of it
    u = oracle.uniform_b200(123, 0, 4096)
    config.manual_seed(123)
    z = Q.act_quantized_dropout(torch.ones(4096, device="cuda"), 0.3, True)
    assert np.array_equal(z.cpu().numpy() != 0, u > np.float32(0.3))


def test_dropout_eval_returns_input():
    x = torch.randn(10, 10, device="cuda")
    assert Q.act_quantized_dropout(x, 0.5, False) is x   # quantization.cc:115-117


@pytest.mark.parametrize("p", [0.5, 0.2])
@pytest.mark.parametrize("shape", [(2330, 602), (1001, 7), (5,)])
def test_relu_dropout_in_one_pass_equals_the_two_ops(shape, p):
    """exact_act_quantized_relu_dropout_forward: outputs and gradients bit-identical to act_quantized_relu
    followed by act_quantized_dropout, with supplied uniforms and with the Philox draw of the same offset."""
    from exact_b200 import config
    x = np.random.default_rng(3).standard_normal(shape).astype(np.float32)
    u = uniform01(shape, 4)
    g = np.random.default_rng(5).standard_normal(shape).astype(np.float32)
    for uniforms in (torch.from_numpy(u).cuda(), None):
        outs = []
        for fused in (True, False):
            config.manual_seed(77)
            xt = torch.from_numpy(x).cuda().requires_grad_()
            if fused:
                y = Q.act_quantized_relu_dropout(xt, p, True, uniforms=uniforms)
            else:
                y = Q.act_quantized_dropout(Q.act_quantized_relu(xt), p, True, uniforms=uniforms)
            y.backward(torch.from_numpy(g).cuda())
            outs.append((y.detach().clone(), xt.grad.clone()))
        assert torch.equal(outs[0][0], outs[1][0]) and torch.equal(outs[0][1], outs[1][1])
    # and against the oracle's two steps
    out, keep = oracle.dropout_fw(oracle.relu_fw(x)[0], u, p)
    xt = torch.from_numpy(x).cuda()
    y = Q.act_quantized_relu_dropout(xt, p, True, uniforms=torch.from_numpy(u).cuda())
    assert np.array_equal(y.cpu().numpy(), out)
    assert torch.equal(Q.act_quantized_relu_dropout(xt, p, False), torch.relu(xt))


def test_leaky_relu_equals_torch_exactly():
    """test/test_op.py:165-184: output and gradient equal F.leaky_relu(0.2) exactly (10,000 x 128), plus an
    unaligned view and a length that is not a multiple of 128."""
    import torch.nn.functional as F
    from exact_b200.cpp_extension import quantization as Q
    for shape, view in (((10000, 128), False), ((777, 13), False), ((1000, 64), True)):
        g = torch.Generator(device="cuda").manual_seed(5)
        x = torch.randn(*shape, device="cuda", generator=g)
        if view:
            x = torch.randn(shape[0] * shape[1] + 1, device="cuda", generator=g)[1:].view(*shape)
        go = torch.randn(*shape, device="cuda", generator=g)
        a = x.clone().requires_grad_()
        b = x.clone().requires_grad_()
        ya = Q.act_quantized_leaky_relu(a, 0.2)
        yb = F.leaky_relu(b, 0.2)
        ya.backward(go)
        yb.backward(go)
        assert torch.equal(ya, yb) and torch.equal(a.grad, b.grad)
