"""GPU parity of the fused projection + quantise + pack kernel (TMA + tcgen05) against the oracle.

Criteria: (i) the projection the epilogue saw agrees with the fp32 product within 1e-2 relative
Frobenius (tf32 inputs); (ii) given those values, the row statistics and the packed stream are
bit-exact against the oracle fed with the same values and the restated noise; (iii) the status word
stays 0 (no bounded wait expired)."""
import numpy as np
import pytest
import torch

import oracle
from exact_b200 import config
from exact_b200.cpp_extension import quantization as Q
from helpers import normal

pytestmark = pytest.mark.gpu

CASES = [
    # N, D, k, bits
    (256, 128, 32, 2), (128, 32, 16, 2), (1000, 256, 32, 2), (1000, 100, 13, 2), (777, 256, 76, 2),
    (4096, 128, 64, 1), (4096, 128, 16, 4), (513, 64, 8, 8), (300, 512, 128, 2), (50000, 256, 32, 2),
    (130, 1024, 256, 2), (9, 36, 5, 2),
    # rows that are not 16-byte aligned (cp.async producers): the reddit-shaped 602 features, odd D (4-byte pieces)
    (64, 602, 76, 2), (5000, 602, 76, 2), (1000, 602, 76, 4), (333, 37, 5, 2), (2000, 101, 13, 8), (129, 602, 76, 1),
    # k beyond one MMA: two MMAs per K step, one accumulator buffer
    (700, 602, 301, 2), (1000, 1024, 512, 2), (300, 640, 320, 4),
]


def rel_fro(a, b):
    a, b = a.astype(np.float64), b.astype(np.float64)
    return np.linalg.norm(a - b) / (np.linalg.norm(b) + 1e-30)


@pytest.mark.parametrize("N,D,k,bits", CASES)
def test_fused_projection_pack(N, D, k, bits):
    config.check_device_status = True
    x = normal(N, D, 1)
    seed, off_r, off_n = 21, 3, 4
    R = oracle.rademacher(seed, off_r, D, k)
    xt, Rt = torch.from_numpy(x).cuda(), torch.from_numpy(R).cuda()
    packed, sb, mb, y = Q.rp_quantize_pack(xt, Rt, bits, seed=seed, offset=off_n, row_offset=0, want_projection=True)
    y = y.cpu().numpy()
    ref_y = oracle.input2rp(x, R)
    assert rel_fro(y, ref_y) < 1e-2                       # (i)
    assert rel_fro(y, ref_y) < 3e-3                       # tf32 truncation of x is about 1e-3
    noise = oracle.noise_b200_rows(seed, off_n, N, k)
    op, osb, omb, _, _ = oracle.quantize_activation(y, noise, bits)
    assert np.array_equal(sb.view(torch.int16).cpu().numpy().view(np.uint16), osb)      # (ii)
    assert np.array_equal(mb.view(torch.int16).cpu().numpy().view(np.uint16), omb)
    assert np.array_equal(packed.cpu().numpy().view(np.uint8)[:-1], op)
    # without the debugging copy of the projection the epilogue takes its conversion-free path on full
    # tiles: same bytes
    packed2, sb2, mb2 = Q.rp_quantize_pack(xt, Rt, bits, seed=seed, offset=off_n, row_offset=0)
    assert torch.equal(packed2[:-1], packed[:-1]) and torch.equal(sb2, sb) and torch.equal(mb2, mb)
    config.check_device_status = False


def test_unsupported_shapes_are_refused():
    x = torch.randn(64, 1200, device="cuda")
    R = torch.randn(1200, 600, device="cuda")         # more accumulator columns than TMEM has
    with pytest.raises(RuntimeError):
        Q.rp_quantize_pack(x, R, 2)
    assert not Q.rp_supported(1200, 600)
    assert Q.rp_supported(602, 76) and Q.rp_supported(602, 301) and Q.rp_supported(256, 32) and Q.rp_supported(37, 5)


def test_rows_of_a_view_that_is_not_16_byte_aligned():
    """A [N, 128] matrix that starts 8 bytes into its storage takes the cp.async route and gives the bytes of
    the aligned call."""
    N, D, k, bits = 3000, 128, 16, 2
    x = normal(N, D, 7)
    R = torch.from_numpy(oracle.rademacher(3, 0, D, k)).cuda()
    base = torch.zeros(N * D + 2, device="cuda")
    view = base[2:].view(N, D)
    view.copy_(torch.from_numpy(x))
    assert view.data_ptr() % 16 == 8
    a = Q.rp_quantize_pack(torch.from_numpy(x).cuda(), R, bits, seed=1, offset=2, row_offset=0)
    b = Q.rp_quantize_pack(view, R, bits, seed=1, offset=2, row_offset=0)
    assert torch.equal(a[0][:-1], b[0][:-1])          # the last byte is allocated and never written
    assert torch.equal(a[1].view(torch.int16), b[1].view(torch.int16))
    assert torch.equal(a[2].view(torch.int16), b[2].view(torch.int16))


BWD_CASES = [(256, 128, 32, 2), (1000, 256, 32, 2), (1000, 100, 13, 2), (4096, 128, 16, 4), (513, 64, 8, 8),
             (50000, 256, 32, 2), (130, 256, 64, 1), (9, 36, 5, 2), (3000, 200, 25, 2),
             # sign(R) not resident: streamed in panels, output in column blocks
             (20000, 256, 128, 2), (5000, 602, 76, 2), (3000, 602, 301, 2), (1000, 602, 76, 8), (700, 300, 37, 4),
             (129, 1030, 33, 1), (40000, 602, 76, 4)]


@pytest.mark.parametrize("N,D,k,bits", BWD_CASES)
def test_fused_unpack_transpose_projection(N, D, k, bits):
    """dequantise(packed) @ R^T in one kernel against the oracle's dequantise -> rp2input
    (ops.py:164-166): 1e-2 relative Frobenius (tf32 rounding of the dequantised values)."""
    config.check_device_status = True
    y = normal(N, k, 5)
    noise = oracle.noise_b200(1, 2, N, k)
    op, osb, omb, _, _ = oracle.quantize_activation(y, noise, bits)
    R = oracle.rademacher(7, 1, D, k)
    ref = oracle.rp2input(oracle.dequantize_activation(op, osb, omb, N, k, bits), R)
    pk = torch.from_numpy(np.concatenate([op, np.zeros(3, np.uint8)]).view(np.int8)).cuda()
    sb = torch.from_numpy(osb.view(np.int16)).cuda().view(torch.bfloat16)
    mb = torch.from_numpy(omb.view(np.int16)).cuda().view(torch.bfloat16)
    out = Q.unpack_dequant_rp(pk, bits, sb, mb, N, torch.from_numpy(R).cuda()).cpu().numpy()
    assert out.shape == (N, D)
    assert rel_fro(out, ref) < 1e-2
    assert rel_fro(out, ref) < 3e-3
    config.check_device_status = False


@pytest.mark.parametrize("N,D,k", [(5000, 256, 32), (3000, 602, 76), (2000, 100, 13), (500, 128, 16)])
def test_public_input2rp_and_rp2input_against_the_oracle(N, D, k):
    """ops.input2rp / ops.rp2input (exact/exact/ops.py:107-125), the unfused projection pair: dense products on this
    library's tensor-core GEMM from 1,024 rows on (tf32 head/tail split: fp32-class accuracy), the library's
    otherwise; against the oracle's double-accumulated products."""
    from exact_b200 import ops
    config.manual_seed(21)
    x = normal(N, D, 41)
    y, R = ops.input2rp(torch.from_numpy(x).cuda(), k)
    Rn = R.cpu().numpy()
    assert np.array_equal(np.abs(Rn), np.full_like(Rn, 1.0 / np.sqrt(np.float32(k))))
    assert rel_fro(y.cpu().numpy(), oracle.input2rp(x, Rn)) < 1e-5
    back = ops.rp2input(y, torch.Size([N, D]), R)
    assert rel_fro(back.cpu().numpy(), oracle.rp2input(y.cpu().numpy(), Rn)) < 1e-5
