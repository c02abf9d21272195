"""Dense-layer GEMM on the tensor cores with operands split into tf32 head and tail
(exact_linear_forward) against an fp64 product, over every shape class the layers use (ragged K and N,
second operand pair, accumulation into C, outputs wider than one MMA tile).

Accuracy bar.  The split products are exact to about 2^-22; what remains is the tensor core's fp32
accumulator, which truncates instead of rounding, once per MMA (three MMAs per 8 columns of K), so the
error grows linearly with K: measured 0.8e-6 (K = 100) and 1.9e-6 (K = 256) relative Frobenius error
against fp64, where the library's fp32 SIMT GEMM has 2e-7 .. 3e-7 and a single-pass tf32 GEMM 5e-4.
The bound used here is 5e-7 + 1e-8 K."""
import numpy as np
import pytest
import torch

from exact_b200 import config
from exact_b200.cpp_extension import backward_func as B
from helpers import normal

pytestmark = pytest.mark.gpu


def relfro(a, b):
    return float((a.double() - b.double()).norm() / b.double().norm())


def t(a):
    return torch.from_numpy(a).cuda()


def tol(K):
    return 5e-7 + 1e-8 * K


@pytest.mark.parametrize("M,K,N", [(3000, 256, 256), (5000, 100, 256), (4097, 256, 47), (2048, 48, 256),
                                   (1500, 47, 256), (1300, 256, 300), (1111, 602, 16), (1024, 8, 8)])
@pytest.mark.parametrize("with_bias", [False, True])
def test_linear_forward_matches_fp64(M, K, N, with_bias):
    a, w = t(normal(M, K, 1)), t(normal(N, K, 2))
    b = t(normal(1, N, 3)).reshape(N) if with_bias else None
    ref = a.double() @ w.double().t()
    if with_bias:
        ref = ref + b.double()
    out = B.linear_forward(a, w, b)
    lib = torch.nn.functional.linear(a, w, b)
    e_out, e_lib = relfro(out, ref), relfro(lib, ref)
    assert out.shape == (M, N) and out.dtype == torch.float32
    assert e_lib < 5e-7
    assert e_out < tol(K), (e_out, e_lib)
    # elementwise: relative to sum_k |a||w|, the natural scale of a dot product's rounding error
    scale = a.double().abs() @ w.double().abs().t() + 1e-30
    assert float(((out.double() - ref).abs() / scale).max()) < tol(K)


def test_two_operand_pairs_bias_and_accumulate():
    M, K1, K2, N = 2500, 256, 100, 256
    a1, a2 = t(normal(M, K1, 1)), t(normal(M, K2, 2))
    w1, w2, b = t(normal(N, K1, 3)), t(normal(N, K2, 4)), t(normal(1, N, 5)).reshape(N)
    ref = a1.double() @ w1.double().t() + a2.double() @ w2.double().t() + b.double()
    out = B.linear_forward(a1, w1, b, a2=a2, weight2=w2)
    assert relfro(out, ref) < tol(K1 + K2)
    c0 = t(normal(M, N, 6))
    c = c0.clone()
    r = B.linear_forward(a1, w1, None, out=c, accumulate=True)
    assert r.data_ptr() == c.data_ptr()
    assert relfro(c, c0.double() + a1.double() @ w1.double().t()) < tol(K1)


def test_strided_rows_and_column_block_of_c():
    """Row pitches larger than the rows (lda, ldc) and a transposed weight view."""
    M, K, N = 2000, 64, 32
    big = t(normal(M, 128, 1))
    a = big[:, 32:96]                      # pitch 128, 16-byte aligned start
    w = t(normal(K, N, 2)).t()             # [N, K] view with stride(1) != 1
    cbig = torch.zeros(M, 96, device="cuda")
    B.linear_forward(a, w, None, out=cbig[:, 64:96])
    assert relfro(cbig[:, 64:96], a.double() @ w.double().t()) < tol(K)
    assert float(cbig[:, :64].abs().max()) == 0.0


def test_non_finite_inputs_stay_local():
    """A row holding inf or NaN comes out non-finite (the tail of inf is inf - inf = NaN); every other row
    is unaffected."""
    M, K, N = 1536, 64, 48
    a, w = t(normal(M, K, 1)), t(normal(N, K, 2))
    a[5, 7] = float("inf")
    a[9, 0] = float("nan")
    out = B.linear_forward(a, w)
    ref = a @ w.t()
    assert torch.isnan(out[9]).all() and not torch.isfinite(out[5]).any()
    keep = torch.ones(M, dtype=torch.bool, device="cuda")
    keep[5] = keep[9] = False
    assert torch.isfinite(out[keep]).all() and relfro(out[keep], ref[keep].double()) < tol(K)


def test_small_or_disabled_uses_library():
    a, w = t(normal(100, 64, 1)), t(normal(32, 64, 2))
    assert torch.equal(B.linear_forward(a, w), torch.nn.functional.linear(a, w))
    a = t(normal(2048, 64, 1))
    config.linear_tensor_core = False
    try:
        assert torch.equal(B.linear_forward(a, w), torch.nn.functional.linear(a, w))
    finally:
        config.linear_tensor_core = True


@pytest.mark.parametrize("M,out,k", [(40037, 64, 32), (70000, 47, 13), (1000, 64, 32)])
def test_rows_reduce_mm(M, out, k):
    """The weight-gradient reduction g^T x (backward_func.cc:87) as a batched product + sum."""
    g, x = t(normal(M, out, 1)), t(normal(M, k, 2))
    ref = g.double().t() @ x.double()
    got = B.rows_reduce_mm(g, x)
    assert got.shape == (out, k) and relfro(got, ref) < 1e-6
