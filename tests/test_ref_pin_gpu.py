"""Pins the oracle (and through it the B200 kernels) to the reference's own unmodified CUDA kernels,
when those have been built into oracle/_ref/ (oracle/build_ref.py).  Skipped otherwise."""
import os
import sys

import numpy as np
import pytest
import torch

import oracle
from helpers import normal, random_csr, relu_normal

pytestmark = pytest.mark.gpu
REF = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "oracle", "_ref")


def _ref(name):
    if not os.path.exists(os.path.join(REF, name + ".so")):
        pytest.skip(f"{name}.so not built (python oracle/build_ref.py)")
    if REF not in sys.path:
        sys.path.insert(0, REF)
    return __import__(name)


@pytest.mark.parametrize("bits", [1, 2, 4, 8])
@pytest.mark.parametrize("shape", [(4096, 128), (37, 13), (131, 76), (50, 602), (1000, 256)])
def test_reference_pack_unpack_equal_oracle(shape, bits):
    rq = _ref("ref_quantization")
    N, D = shape
    x = relu_normal(N, D, 101)
    xt = torch.from_numpy(x).cuda()
    mn, mx = xt.min(1)[0], xt.max(1)[0]
    scale = (2 ** bits - 1) / (mx - mn)
    torch.manual_seed(1234 + bits)
    offset = int(torch.cuda.default_generators[torch.cuda.current_device()].get_offset())
    packed = rq.pack_single_precision(xt, mn, mx, scale, bits, True)
    torch.cuda.synchronize()
    omn, omx, osc = oracle.row_stats(x, bits)
    assert np.array_equal(scale.cpu().numpy().view(np.int32), osc.view(np.int32))
    noise = oracle.noise_reference_pack(1234 + bits, offset, N, D, bits)
    ours = oracle.pack(x, omn, osc, noise, bits, use_fma=True)
    ref = packed.cpu().numpy().view(np.uint8)[:-1]
    assert np.array_equal(ref, ours)
    sb, mb = scale.to(torch.bfloat16), mn.to(torch.bfloat16)
    up = rq.unpack_single_precision(packed, bits, sb.float(), mb.float(), N, D)
    ref_up = oracle.unpack(ours, oracle.bf16_to_f32(oracle.f32_to_bf16(osc)),
                           oracle.bf16_to_f32(oracle.f32_to_bf16(omn)), N, D, bits)
    assert np.array_equal(up.cpu().numpy(), ref_up)


@pytest.mark.parametrize("bits", [1, 2, 4, 8])
@pytest.mark.parametrize("shape", [(4096, 128), (37, 13), (131, 76), (1000, 256)])
def test_reference_half_pack_unpack_equal_oracle(shape, bits):
    """The half instantiations of the reference's kernels (quantization_cuda_kernel.cu:132, 209) and torch's
    half tensor ops for the statistics (ops.py:63, 39) against the fp16 oracle, bit for bit."""
    rq = _ref("ref_quantization")
    N, D = shape
    x = (normal(N, D, 303) * 2.5).astype(np.float16)
    xt = torch.from_numpy(x).cuda()
    mn, mx = xt.min(1)[0], xt.max(1)[0]
    scale = (2 ** bits - 1) / (mx - mn)
    torch.manual_seed(4321 + bits)
    offset = int(torch.cuda.default_generators[torch.cuda.current_device()].get_offset())
    packed = rq.pack_single_precision(xt, mn, mx, scale, bits, True)
    torch.cuda.synchronize()
    noise = oracle.noise_reference_pack(4321 + bits, offset, N, D, bits)
    op, osc, omn = oracle.quantize_activation_f16(x, noise, bits)
    assert np.array_equal(scale.cpu().numpy().view(np.uint16), osc.view(np.uint16))
    assert np.array_equal(mn.cpu().numpy().view(np.uint16), omn.view(np.uint16))
    assert np.array_equal(packed.cpu().numpy().view(np.uint8)[:-1], op)
    up = rq.unpack_single_precision(packed, bits, scale, mn, N, D)
    assert up.dtype == torch.float16
    assert np.array_equal(up.cpu().numpy().view(np.uint16), oracle.unpack_f16(op, osc, omn, N, D, bits).view(np.uint16))


@pytest.mark.parametrize("reduce", ["sum", "mean"])
@pytest.mark.parametrize("with_values", [True, False])
def test_reference_half_spmm_equals_oracle(with_values, reduce):
    """The half instantiation of the reference's SpMM kernel (spmm_cuda.cu:142) against the fp16 oracle."""
    rs = _ref("ref_spmm")
    n, K = 3000, 72
    rowptr, col, val = random_csr(n, n, 40000, 31, with_values=True)
    valh = (val * 0.5).astype(np.float16) if with_values else None
    mat = normal(n, K, 32).astype(np.float16)
    t = lambda a: torch.from_numpy(a).cuda()
    v = None if valh is None else t(valh)
    if reduce == "sum":
        out = rs.spmm_sum_fw(None, t(rowptr), t(col), v, None, None, t(mat))
    else:
        out = rs.spmm_mean_fw(None, t(rowptr), t(col), v, None, None, None, t(mat))
    ref = oracle.spmm_f16(rowptr, col, valh, mat, reduce)
    assert np.array_equal(out.cpu().numpy().view(np.uint16), ref.view(np.uint16))


def test_fma_contraction_in_reference_pack():
    """quantization_cuda_kernel.cu:89 is compiled with nvcc's default -fmad=true.  On an input large
    enough for the two variants to differ, the reference's binary must match the FMA variant of the
    oracle and not the uncontracted one."""
    rq = _ref("ref_quantization")
    N, D, bits = 40000, 256, 8
    x = relu_normal(N, D, 202)
    xt = torch.from_numpy(x).cuda()
    mn, mx = xt.min(1)[0], xt.max(1)[0]
    scale = (2 ** bits - 1) / (mx - mn)
    torch.manual_seed(99)
    offset = int(torch.cuda.default_generators[torch.cuda.current_device()].get_offset())
    ref = rq.pack_single_precision(xt, mn, mx, scale, bits, True).cpu().numpy().view(np.uint8)[:-1]
    omn, omx, osc = oracle.row_stats(x, bits)
    noise = oracle.noise_reference_pack(99, offset, N, D, bits)
    fma = oracle.pack(x, omn, osc, noise, bits, use_fma=True)
    nofma = oracle.pack(x, omn, osc, noise, bits, use_fma=False)
    assert np.array_equal(ref, fma)
    if not np.array_equal(fma, nofma):
        assert not np.array_equal(ref, nofma)
    print("bytes on which the two variants differ:", int((fma != nofma).sum()))


@pytest.mark.parametrize("reduce", ["sum", "mean"])
@pytest.mark.parametrize("with_values", [True, False])
def test_reference_spmm_equals_oracle(reduce, with_values):
    rs = _ref("ref_spmm")
    rowptr, col, val = random_csr(10000, 10000, 50000, 3, with_values)
    mat = normal(10000, 128, 4)
    t = lambda a: torch.from_numpy(a).cuda()
    v = t(val) if with_values else None
    if reduce == "sum":
        out = rs.spmm_sum_fw(None, t(rowptr), t(col), v, None, None, t(mat))
    else:
        out = rs.spmm_mean_fw(None, t(rowptr), t(col), v, None, None, None, t(mat))
    assert np.array_equal(out.cpu().numpy(), oracle.spmm(rowptr, col, val, mat, reduce))


@pytest.mark.parametrize("reduce", ["sum", "mean"])
def test_reference_value_gradient_equals_oracle(reduce):
    """spmm_sum_bw / spmm_mean_bw with value_requires_grad (spmm.cc:57-79, 115-139 -> spmm_value_bw_kernel)."""
    rs = _ref("ref_spmm")
    n, K = 4000, 100
    rowptr, col, val = random_csr(n, n, 30000, 3, True)
    row = np.repeat(np.arange(n), np.diff(rowptr))
    mat, g = normal(n, K, 4), normal(n, K, 5)
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    perm = np.argsort(col * n + row, kind="stable")
    colptr = np.zeros(n + 1, np.int64)
    np.cumsum(np.bincount(col, minlength=n), out=colptr[1:])
    args = [t(row), t(rowptr), t(col), t(val)]
    if reduce == "mean":
        args.append(t(np.diff(rowptr)))
    args += [t(colptr), t(perm), t(mat), t(g), True, True, False]
    fn = rs.spmm_sum_bw if reduce == "sum" else rs.spmm_mean_bw
    grad_value = fn(*args)[0]
    assert np.array_equal(grad_value.cpu().numpy(), oracle.spmm_value_bw(rowptr, col, mat, g, reduce))


@pytest.mark.parametrize("reduce", ["max", "min"])
@pytest.mark.parametrize("with_values", [True, False])
def test_reference_max_min_equal_oracle(reduce, with_values):
    rs = _ref("ref_spmm")
    rowptr, col, val = random_csr(4000, 4000, 20000, 3, with_values)
    mat = normal(4000, 64, 4)
    mat[:, 0] = 1.0     # ties: the first edge of a row must win
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    fn = rs.spmm_max_fw if reduce == "max" else rs.spmm_min_fw
    out, arg = fn(t(rowptr), t(col), t(val) if with_values else None, t(mat))
    ref_out, ref_arg = oracle.spmm_minmax(rowptr, col, val, mat, reduce)
    assert np.array_equal(out.cpu().numpy(), ref_out)
    assert np.array_equal(arg.cpu().numpy(), ref_arg)
