"""fp16 activations (the AMP path of the reference: exact/exact/ops.py:82-83, 130; half instantiations of the pack /
unpack kernels, quantization_cuda_kernel.cu:132, 209): the CUDA kernels against the fp16 oracle, bit for bit."""
import numpy as np
import pytest
import torch

import oracle
from exact_b200 import config, ops
from exact_b200.cpp_extension import quantization as Q
from helpers import normal, uniform01

pytestmark = pytest.mark.gpu

SHAPES = [(4096, 128), (37, 13), (131, 76), (9, 602), (1000, 256), (8, 1), (1, 7)]


def _half(N, D, seed):
    x = (normal(N, D, seed) * 2.5).astype(np.float16)
    if N > 3:
        x[3] = x[3, 0]          # a constant row: scale = inf, codes 0, dequantised = min
    return x


@pytest.mark.parametrize("bits", [1, 2, 4, 8])
@pytest.mark.parametrize("N,D", SHAPES)
def test_quantize_pack_and_unpack_f16_bit_exact(N, D, bits):
    x = _half(N, D, 5)
    noise = uniform01((N, D), 6)
    op, osc, omn = oracle.quantize_activation_f16(x, noise, bits)
    xt = torch.from_numpy(x).cuda()
    pk, sc, mn = Q.quantize_pack(xt, bits, noise=torch.from_numpy(noise).cuda())
    assert sc.dtype == torch.float16 and mn.dtype == torch.float16
    assert np.array_equal(sc.cpu().numpy().view(np.uint16), osc.view(np.uint16))
    assert np.array_equal(mn.cpu().numpy().view(np.uint16), omn.view(np.uint16))
    assert np.array_equal(pk.cpu().numpy().view(np.uint8)[:-1], op)
    out = Q.unpack_single_precision(pk, bits, sc, mn, N, D)
    assert out.dtype == torch.float16 and out.shape == (N, D)
    ref = oracle.unpack_f16(op, osc, omn, N, D, bits)
    got = out.cpu().numpy()
    both_nan = np.isnan(got) & np.isnan(ref)
    assert np.array_equal(got.view(np.uint16)[~both_nan], ref.view(np.uint16)[~both_nan])
    # the reference signature with caller-computed half statistics
    pk2 = Q.pack_single_precision(xt, mn, mn, sc, bits, True, noise=torch.from_numpy(noise).cuda())
    assert np.array_equal(pk2.cpu().numpy().view(np.uint8)[:-1], op)


@pytest.mark.parametrize("bits", [2, 8])
def test_production_noise_f16_matches_the_restated_stream(bits):
    N, D = 1003, 76
    x = _half(N, D, 7)
    pk, sc, mn = Q.quantize_pack(torch.from_numpy(x).cuda(), bits, seed=17, offset=3, row_offset=16)
    noise = oracle.noise_b200(17, 3, N, D, row_offset=16)
    op, osc, omn = oracle.quantize_activation_f16(x, noise, bits)
    assert np.array_equal(pk.cpu().numpy().view(np.uint8)[:-1], op)


def test_quantize_and_dequantize_activation_keep_fp16():
    """ops.py:69-98 on an fp16 activation: fp16 statistics in, fp16 reconstruction out, error within one
    quantisation step."""
    config.manual_seed(3)
    config.compress_activation, config.simulate, config.activation_compression_bits = True, False, [2]
    x = torch.from_numpy(_half(2000, 64, 9)).cuda()
    q = ops.quantize_activation(x, None)
    assert q[2].dtype == torch.float16 and q[3].dtype == torch.float16
    xh = ops.dequantize_activation(q, x.shape)
    assert xh.dtype == torch.float16 and xh.shape == x.shape
    step = (x.float().max(1)[0] - x.float().min(1)[0]) / (2 ** config.activation_compression_bits[0] - 1)
    # one quantisation step plus the half roundings of x - min, code / scale and + min (values up to 16: 2^-6 each).
    # Not every element: the reference's pack has no upper clamp (quantization_cuda_kernel.cu:89-90), and a row
    # maximum whose half-rounded scale puts it a hair above 2^bits - 1 rounds up to 2^bits with noise near 1; that
    # code then spills into the next row's field, here as in the reference's half kernel.
    bad = (xh.float() - x.float()).abs() > 1.02 * step[:, None] + 5e-2
    assert float(bad.float().mean()) < 2e-3


def test_mask_activations_on_fp16():
    """ReLU, LeakyReLU, dropout and ReLU + dropout on halves: the fp32 arithmetic of the oracle on widened values,
    rounded to half once (Half (op) float is a float in the reference's half kernels), forward and backward."""
    n = 128 * 37 + 5
    x = (normal(1, n, 11)[0] * 2).astype(np.float16)
    g = (normal(1, n, 12)[0]).astype(np.float16)
    u = uniform01((n,), 13)
    xt = torch.from_numpy(x).cuda().requires_grad_()
    gt = torch.from_numpy(g).cuda()
    ut = torch.from_numpy(u).cuda()
    xf, gf = x.astype(np.float32), g.astype(np.float32)

    y = Q.act_quantized_relu(xt)
    (gx,) = torch.autograd.grad(y, xt, gt)
    assert y.dtype == torch.float16 and np.array_equal(y.detach().cpu().numpy(), np.maximum(x, 0))
    assert np.array_equal(gx.cpu().numpy(), np.where(x > 0, g, np.float16(0)))

    slope = 0.01
    y = Q.act_quantized_leaky_relu(xt, slope)
    (gx,) = torch.autograd.grad(y, xt, gt)
    ref = np.where(xf > 0, xf, xf * np.float32(slope)).astype(np.float16)
    assert np.array_equal(y.detach().cpu().numpy().view(np.uint16), ref.view(np.uint16))
    refg = np.where(xf > 0, gf, gf * np.float32(slope)).astype(np.float16)
    assert np.array_equal(gx.cpu().numpy().view(np.uint16), refg.view(np.uint16))

    p = 0.3
    y = Q.act_quantized_dropout(xt, p, True, uniforms=ut)
    (gx,) = torch.autograd.grad(y, xt, gt)
    out, keep = oracle.dropout_fw(xf, u, p)
    assert np.array_equal(y.detach().cpu().numpy().view(np.uint16), out.astype(np.float16).view(np.uint16))
    assert np.array_equal(gx.cpu().numpy().view(np.uint16), oracle.dropout_bw(gf, keep, p).astype(np.float16).view(np.uint16))

    y = Q.act_quantized_relu_dropout(xt, p, True, uniforms=ut)
    (gx,) = torch.autograd.grad(y, xt, gt)
    r, rk = oracle.relu_fw(xf)
    out, keep = oracle.dropout_fw(r, u, p)
    assert np.array_equal(y.detach().cpu().numpy().view(np.uint16), out.astype(np.float16).view(np.uint16))
    refg = oracle.mask_bw(oracle.dropout_bw(gf, keep, p), rk).astype(np.float16)
    assert np.array_equal(gx.cpu().numpy().view(np.uint16), refg.view(np.uint16))


@pytest.mark.parametrize("idx", [torch.int64, torch.int32])
@pytest.mark.parametrize("reduce", ["sum", "mean"])
@pytest.mark.parametrize("with_values", [True, False])
@pytest.mark.parametrize("K", [128, 100, 13, 256])
def test_spmm_f16_bit_exact(K, with_values, reduce, idx):
    """SpMM on halves: every product and partial sum rounded to half in CSR order, the mean's divisor rounded to
    half first (a hub row of 3000 edges: half(3000) = 3000, of 5001: 5000), against the fp16 oracle."""
    from exact_b200.cpp_extension import spmm as S
    from helpers import random_csr
    n = 6000
    rowptr, col, val = random_csr(n, n, 60000, 21, with_values=True)
    rng = np.random.default_rng(22)
    hub = np.sort(rng.choice(n, 5001, replace=False))
    # replace row 7 by a hub row whose length half precision cannot represent
    keep = np.repeat(np.arange(n), np.diff(rowptr)) != 7
    row = np.concatenate([np.repeat(np.arange(n), np.diff(rowptr))[keep], np.full(5001, 7)])
    colx = np.concatenate([col[keep], hub])
    valx = np.concatenate([val[keep], rng.standard_normal(5001).astype(np.float32)])
    order = np.argsort(row * n + colx, kind="stable")
    row, colx, valx = row[order], colx[order], valx[order]
    rowptr = np.zeros(n + 1, np.int64)
    np.cumsum(np.bincount(row, minlength=n), out=rowptr[1:])
    valh = (valx * 0.5).astype(np.float16) if with_values else None
    mat = (normal(n, K, 23)).astype(np.float16)
    ref = oracle.spmm_f16(rowptr, colx, valh, mat, reduce)
    out = S._spmm(torch.from_numpy(rowptr).to(idx).cuda(), torch.from_numpy(colx).to(idx).cuda(),
                  None if valh is None else torch.from_numpy(valh).cuda(), torch.from_numpy(mat).cuda(), reduce)
    assert out.dtype == torch.float16
    assert np.array_equal(out.cpu().numpy().view(np.uint16), ref.view(np.uint16))
