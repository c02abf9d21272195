"""Batch-norm backward read straight from the packed input (exact_bn_backward_from_packed) against the oracle:
dequantize_activation (bit-exact restatement) followed by native_batch_norm_backward in float64, and against
ATen's own backward fed the dequantised tensor (the reference's chain, exact/exact/ops.py:235-253)."""
import numpy as np
import pytest
import torch

import oracle
from exact_b200 import config
from exact_b200.cpp_extension import backward_func as B
from exact_b200.cpp_extension import quantization as Q
from helpers import normal

pytestmark = pytest.mark.gpu


def _case(N, D, bits, seed):
    x = normal(N, D, seed) * 1.7 + 0.3
    noise = oracle.noise_b200(3, 5, N, D)
    op, osb, omb, _, _ = oracle.quantize_activation(x, noise, bits)
    xhat = oracle.dequantize_activation(op, osb, omb, N, D, bits)
    pk = torch.from_numpy(np.concatenate([op, np.zeros(3, np.uint8)]).view(np.int8)).cuda()
    sb = torch.from_numpy(osb.view(np.int16)).cuda().view(torch.bfloat16)
    mb = torch.from_numpy(omb.view(np.int16)).cuda().view(torch.bfloat16)
    return x, xhat, (pk, bits, sb, mb)


@pytest.mark.parametrize("training", [True, False])
@pytest.mark.parametrize("bits", [1, 2, 4, 8])
@pytest.mark.parametrize("N,D", [(21168, 256), (1000, 128), (1003, 100), (37, 4), (3000, 1028), (8, 64)])
def test_bn_backward_from_packed(N, D, bits, training):
    x, xhat, quantized = _case(N, D, bits, 40 + bits)
    g = normal(N, D, 50)
    rng = np.random.default_rng(60)
    w = rng.standard_normal(D).astype(np.float32)
    rm = rng.standard_normal(D).astype(np.float32) * 0.1
    rv = (rng.random(D) + 0.5).astype(np.float32)
    eps = 1e-5
    xt, gt = torch.from_numpy(x).cuda(), torch.from_numpy(g).cuda()
    wt, rmt, rvt = (torch.from_numpy(a).cuda() for a in (w, rm, rv))
    # statistics of the forward on the exact input, as qbatch_norm.forward saves them (ops.py:212-226)
    _, save_mean, save_invstd = torch.ops.aten.native_batch_norm(xt, wt, None, rmt.clone(), rvt.clone(), training, 0.1, eps)
    assert B.batch_norm_backward_from_packed_supported(gt, quantized)
    gi, gw, gb = B.batch_norm_backward_from_packed(gt, quantized, wt, rmt, rvt, save_mean, save_invstd, training, eps,
                                                   [True, True, True])
    if training:
        mean, invstd = save_mean.cpu().numpy(), save_invstd.cpu().numpy()
    else:
        mean, invstd = rm, 1.0 / np.sqrt(rv.astype(np.float64) + eps)
    ri, rw, rb = oracle.bn_backward(g, xhat, w, mean, invstd, training)
    # fp32 sums over N rows against float64: a few ulps times sqrt(N) of the summands' scale
    s_scale = np.sqrt(N) * 4e-6
    assert np.all(np.abs(gb.cpu().numpy() - rb) <= s_scale * np.abs(g).max() + 1e-6 * np.abs(rb))
    gx_scale = (np.abs(g) * np.abs(xhat - mean[None, :])).max() * np.abs(invstd).max()
    assert np.all(np.abs(gw.cpu().numpy() - rw) <= s_scale * gx_scale + 1e-6 * np.abs(rw))
    err = np.abs(gi.cpu().numpy() - ri)
    assert err.max() <= 2e-5 * np.abs(ri).max() + 1e-6
    # ... and no further from float64 than ATen's own backward on the dequantised tensor
    ai, aw, ab = torch.ops.aten.native_batch_norm_backward(gt, torch.from_numpy(xhat).cuda(), wt, rmt, rvt, save_mean,
                                                           save_invstd, training, eps, [True, True, True])
    assert err.max() <= 4 * np.abs(ai.cpu().numpy() - ri).max() + 1e-6 * np.abs(ri).max()
    # run-to-run identical (ordered partial sums, no float atomics)
    gi2, gw2, gb2 = B.batch_norm_backward_from_packed(gt, quantized, wt, rmt, rvt, save_mean, save_invstd, training, eps,
                                                      [True, True, True])
    assert torch.equal(gi, gi2) and torch.equal(gw, gw2) and torch.equal(gb, gb2)


def test_bn_backward_output_mask_and_unsupported_width():
    x, xhat, quantized = _case(500, 64, 2, 7)
    g = torch.from_numpy(normal(500, 64, 8)).cuda()
    mean, invstd = torch.zeros(64, device="cuda"), torch.ones(64, device="cuda")
    gi, gw, gb = B.batch_norm_backward_from_packed(g, quantized, None, mean, invstd, mean, invstd, True, 1e-5,
                                                   [True, False, False])
    assert gi is not None and gw is None and gb is None
    gi2, gw2, gb2 = B.batch_norm_backward_from_packed(g, quantized, None, mean, invstd, mean, invstd, True, 1e-5,
                                                      [False, True, True])
    assert gi2 is None and gw2.shape == (64,) and torch.allclose(gb2, g.sum(0), rtol=1e-5, atol=1e-4)
    _, _, q13 = _case(100, 13, 2, 9)
    assert not B.batch_norm_backward_from_packed_supported(torch.zeros(100, 13, device="cuda"), q13)


def test_qbatch_norm_uses_the_packed_backward_and_matches_the_unpacked_route():
    from exact_b200 import ops
    torch.manual_seed(0)
    x = torch.randn(4096, 256, device="cuda", requires_grad=True)
    w = torch.randn(256, device="cuda", requires_grad=True)
    b = torch.randn(256, device="cuda", requires_grad=True)
    g = torch.randn(4096, 256, device="cuda")
    grads = []
    for flag in (True, False):
        config.bn_backward_from_packed = flag
        config.manual_seed(11)
        rm, rv = torch.zeros(256, device="cuda"), torch.ones(256, device="cuda")
        out = ops.qbatch_norm.apply(x, rm, rv, w, b, True, 0.1, 1e-5, None)
        grads.append(torch.autograd.grad(out, (x, w, b), g))
    config.bn_backward_from_packed = True
    for a, c in zip(*grads):
        assert torch.allclose(a, c, rtol=1e-4, atol=1e-4 * float(c.abs().max()))
