"""CPU tests of the oracle itself: it must agree with an independent torch/numpy/scipy statement of
the same reference formulas, and with the golden vectors produced by the reference's own kernels."""
import os

import numpy as np
import pytest
import scipy.sparse as sp
import torch

import oracle
from helpers import normal, random_csr, relu_normal, uniform01

GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "ref_vectors.npz")


def test_philox_known_answers():
    # Random123 known-answer vectors for Philox4x32-10
    assert [hex(v) for v in oracle.philox4x32_10([0, 0, 0, 0], [0, 0])] == \
        ["0x6627e8d5", "0xe169c58d", "0xbc57ac4c", "0x9b00dbd8"]
    assert [hex(v) for v in oracle.philox4x32_10([0xffffffff] * 4, [0xffffffff] * 2)] == \
        ["0x408f276d", "0x41c83b0e", "0xa20bc7c6", "0x6d5451fd"]
    assert [hex(v) for v in oracle.philox4x32_10([0x243f6a88, 0x85a308d3, 0x13198a2e, 0x03707344],
                                                 [0xa4093822, 0x299f31d0])] == \
        ["0xd16cfe09", "0x94fdcceb", "0x5001e420", "0x24126ea1"]


@pytest.mark.parametrize("bits", [1, 2, 4, 8])
def test_row_stats_match_torch(bits):
    # exact/exact/ops.py:61-66 and ops.py:39 evaluated by torch itself on CPU
    x = torch.from_numpy(relu_normal(513, 76, 3))
    mn, mx = torch.min(x, 1)[0], torch.max(x, 1)[0]
    scale = (2 ** bits - 1) / (mx - mn)
    omn, omx, osc = oracle.row_stats(x.numpy(), bits)
    assert np.array_equal(omn, mn.numpy()) and np.array_equal(omx, mx.numpy())
    assert np.array_equal(osc.view(np.int32), scale.numpy().view(np.int32))
    assert np.array_equal(oracle.f32_to_bf16(osc), scale.to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16))


def test_constant_row_gives_inf_scale_and_zero_codes():
    x = np.full((8, 16), 0.25, np.float32)
    u = uniform01((8, 16), 0)
    packed, sb, mb, sf, mf = oracle.quantize_activation(x, u, 2)
    assert np.all(np.isinf(sf)) and np.all(packed == 0)
    xh = oracle.dequantize_activation(packed, sb, mb, 8, 16, 2)
    assert np.array_equal(xh, x)  # 0 / inf + mn


@pytest.mark.parametrize("bits", [1, 2, 4, 8])
@pytest.mark.parametrize("shape", [(4096, 128), (37, 13), (130, 602)])
def test_pack_unpack_against_numpy(bits, shape):
    """quantization_cuda_kernel.cu:73-93 and 167-184 restated with numpy in float32."""
    N, D = shape
    x, u = relu_normal(N, D, 1), uniform01((N, D), 2)
    mn, mx, sc = oracle.row_stats(x, bits)
    packed = oracle.pack(x, mn, sc, u, bits, use_fma=False)
    t = ((x - mn[:, None]) * sc[:, None] + u).astype(np.float32) - np.float32(0.5)
    codes = np.rint(np.maximum(t, 0)).astype(np.int64)
    wpt = 8 // bits
    G = (N + wpt - 1) // wpt
    pad = np.zeros((G * wpt, D), np.int64)
    pad[:N] = codes
    ref = np.zeros((G, D), np.int64)
    for ni in range(wpt):
        ref |= pad[ni::wpt] << (ni * bits)
    assert np.array_equal(packed.reshape(G, D), (ref & 0xff).astype(np.uint8))
    # unpack
    sb, mb = oracle.f32_to_bf16(sc), oracle.f32_to_bf16(mn)
    s32, m32 = oracle.bf16_to_f32(sb), oracle.bf16_to_f32(mb)
    out = oracle.unpack(packed, s32, m32, N, D, bits)
    c2 = np.stack([(packed.reshape(G, D).astype(np.int64) >> (ni * bits)) & (2 ** bits - 1) for ni in range(wpt)], 1)
    c2 = c2.reshape(G * wpt, D)[:N].astype(np.float32)
    assert np.array_equal(out, (c2 / s32[:, None] + m32[:, None]).astype(np.float32))


def test_no_upper_clamp_spills_into_next_field():
    """A code of 2^bits is OR-ed unmasked (quantization_cuda_kernel.cu:90): with INT2, a row-0 code
    of 4 sets bit 2, which belongs to row 1."""
    x = np.zeros((4, 1), np.float32)
    mn = np.zeros(4, np.float32)
    sc = np.ones(4, np.float32)
    x[0, 0] = 3.6
    u = np.full((4, 1), 0.5, np.float32)  # t = 3.6 + 0.5 - 0.5 -> rint 4
    packed = oracle.pack(x, mn, sc, u, 2)
    assert packed[0] == 4


def test_round_trip_error_bound():
    # config 1 of the benchmark: 4096 x 128, INT2
    x, u = relu_normal(4096, 128, 0), uniform01((4096, 128), 1)
    packed, sb, mb, sf, mf = oracle.quantize_activation(x, u, 2)
    xh = oracle.dequantize_activation(packed, sb, mb, 4096, 128, 2)
    step = (x.max(1) - x.min(1)) / 3
    # one quantisation step plus the bf16 rounding of scale/min (2^-8 relative)
    assert np.all(np.abs(xh - x) <= (step * 1.02 + 0.01)[:, None])


def test_relu_matches_torch():
    # test/test_op.py:22-41 (reference asserts equality with F.relu, output and gradient)
    x = normal(1000, 128, 5)
    out, keep = oracle.relu_fw(x)
    xt = torch.from_numpy(x).requires_grad_()
    ref = torch.nn.functional.relu(xt)
    ref.backward(torch.ones_like(ref))
    assert np.array_equal(out, ref.detach().numpy())
    assert np.array_equal(oracle.mask_bw(np.ones_like(x), keep), xt.grad.numpy())


def test_dropout_consistency():
    # test/test_op.py:463-480: zero pattern of output == zero pattern of grad; scale 1/(1-p)
    x = np.ones((2329, 602), np.float32)
    u = uniform01(x.shape, 7)
    out, keep = oracle.dropout_fw(x, u, 0.5)
    g = oracle.dropout_bw(np.ones_like(x), keep, 0.5)
    assert np.array_equal(out == 0, g == 0)
    assert out.max() == 2.0 and g.max() == 2.0
    assert abs(keep.mean() - 0.5) < 0.01


@pytest.mark.parametrize("reduce", ["sum", "mean"])
@pytest.mark.parametrize("with_values", [True, False])
def test_spmm_against_scipy(reduce, with_values):
    # test/test_op.py:506-562 compares with torch_sparse.matmul; scipy is the stand-in here
    rowptr, col, val = random_csr(1000, 1000, 5000, 3, with_values)
    mat = normal(1000, 128, 4)
    out = oracle.spmm(rowptr, col, val, mat, reduce)
    v = np.ones(col.size, np.float32) if val is None else val
    A = sp.csr_matrix((v.astype(np.float64), col, rowptr), shape=(1000, 1000))
    ref = A @ mat.astype(np.float64)
    if reduce == "mean":
        ref = ref / np.maximum(np.diff(rowptr), 1)[:, None]
    np.testing.assert_allclose(out, ref, rtol=1e-5, atol=1e-5)
    # gradient wrt the dense operand == A^T g (sum) or A^T (g / deg) (mean)
    g = normal(1000, 128, 6)
    gm = oracle.spmm_bw_mat(rowptr, col, val, g, 1000, reduce)
    gs = g.astype(np.float64)
    if reduce == "mean":
        gs = gs / np.maximum(np.diff(rowptr), 1)[:, None]
    np.testing.assert_allclose(gm, A.T @ gs, rtol=1e-5, atol=1e-5)


def test_projection_against_numpy():
    x = normal(300, 602, 8)
    R = (2.0 * np.random.default_rng(9).integers(0, 2, (602, 76)) - 1).astype(np.float32) / np.float32(76 ** 0.5)
    y = oracle.input2rp(x, R)
    np.testing.assert_allclose(y, x.astype(np.float64) @ R.astype(np.float64), rtol=1e-6, atol=1e-6)
    xb = oracle.rp2input(y, R)
    np.testing.assert_allclose(xb, y.astype(np.float64) @ R.astype(np.float64).T, rtol=1e-6, atol=1e-6)


@pytest.mark.skipif(not os.path.exists(GOLDEN), reason="golden vectors not generated yet")
def test_oracle_reproduces_reference_kernels():
    """The pin: packed streams, statistics and unpacked values written by the reference's unmodified
    CUDA kernels on a B200 (tests/golden/make_ref_vectors.py) are reproduced bit for bit, with the
    cuRAND noise regenerated from (torch seed, philox offset)."""
    import hashlib
    z = np.load(GOLDEN)
    n_cases = len([k for k in z.files if k.endswith("_meta") and k.startswith("pack")])
    assert n_cases >= 8
    for i in range(n_cases):
        N, D, bits, nseed, tseed, offset = (int(v) for v in z[f"pack{i}_meta"])
        x = relu_normal(N, D, nseed)
        mn, mx, sc = oracle.row_stats(x, bits)
        small = N * D <= 8192
        ref_sc, ref_mn = z[f"pack{i}_scale"], z[f"pack{i}_min"]
        k = ref_sc.size
        assert np.array_equal(sc[:k].view(np.int32), ref_sc.view(np.int32)), f"scale case {i}"
        assert np.array_equal(mn[:k], ref_mn), f"min case {i}"
        noise = oracle.noise_reference_pack(tseed, offset, N, D, bits)
        packed = oracle.pack(x, mn, sc, noise, bits, use_fma=True)
        s32 = oracle.bf16_to_f32(oracle.f32_to_bf16(sc))
        m32 = oracle.bf16_to_f32(oracle.f32_to_bf16(mn))
        up = oracle.unpack(packed, s32, m32, N, D, bits)
        if small:
            assert np.array_equal(packed, z[f"pack{i}_packed"]), f"packed case {i}"
        else:
            assert hashlib.sha256(packed.tobytes()).digest() == z[f"pack{i}_packed"].tobytes(), f"packed case {i}"
        assert hashlib.sha256(up.tobytes()).digest() == z[f"pack{i}_unpacked"].tobytes(), f"unpacked case {i}"
    from golden.make_ref_vectors import SPMM_CASES, make_graph
    for i, (n, K, nnz, seed) in enumerate(SPMM_CASES):
        rowptr, col, val = make_graph(n, nnz, seed)
        mat = np.random.default_rng(seed + 100).standard_normal((n, K)).astype(np.float32)
        for red in ("sum", "mean"):
            for hv in (1, 0):
                out = oracle.spmm(rowptr, col, val if hv else None, mat, red)
                assert hashlib.sha256(out.tobytes()).digest() == z[f"spmm{i}_{red}_{hv}"].tobytes(), \
                    f"spmm case {i} {red} {hv}"


GOLDEN_MORE = os.path.join(os.path.dirname(GOLDEN), "ref_vectors_more.npz")


@pytest.mark.skipif(not os.path.exists(GOLDEN_MORE), reason="second golden fixture not generated yet")
def test_oracle_reproduces_reference_half_kernels_minmax_and_value_gradient():
    """Second fixture written by the reference's unmodified kernels on a B200: the half instantiations of pack /
    unpack / SpMM (statistics from torch's half tensor ops), the max / min aggregation with its winning-edge
    positions and the edge-value gradient, reproduced bit for bit."""
    import hashlib
    from golden.make_ref_vectors import HALF_PACK_CASES, MORE_SPMM_CASES, make_graph, make_half
    z = np.load(GOLDEN_MORE)
    sha = lambda a: hashlib.sha256(np.ascontiguousarray(a).tobytes()).digest()
    for i in range(len(HALF_PACK_CASES)):
        N, D, bits, nseed, tseed, offset = (int(v) for v in z[f"hpack{i}_meta"])
        x = make_half(N, D, nseed)
        noise = oracle.noise_reference_pack(tseed, offset, N, D, bits)
        packed, sc, mn = oracle.quantize_activation_f16(x, noise, bits)
        assert sha(sc.view(np.uint16)) == z[f"hpack{i}_scale"].tobytes(), f"half scale case {i}"
        assert sha(mn.view(np.uint16)) == z[f"hpack{i}_min"].tobytes(), f"half min case {i}"
        assert sha(packed) == z[f"hpack{i}_packed"].tobytes(), f"half packed case {i}"
        up = oracle.unpack_f16(packed, sc, mn, N, D, bits)
        assert sha(up.view(np.uint16)) == z[f"hpack{i}_unpacked"].tobytes(), f"half unpacked case {i}"
    for i, (n, K, nnz, seed) in enumerate(MORE_SPMM_CASES):
        rowptr, col, val = make_graph(n, nnz, seed)
        mat = np.random.default_rng(seed + 100).standard_normal((n, K)).astype(np.float32)
        grad = np.random.default_rng(seed + 200).standard_normal((n, K)).astype(np.float32)
        math, valh = mat.astype(np.float16), (val * 0.5).astype(np.float16)
        for red in ("sum", "mean"):
            for hv in (1, 0):
                out = oracle.spmm_f16(rowptr, col, valh if hv else None, math, red)
                assert sha(out.view(np.uint16)) == z[f"hspmm{i}_{red}_{hv}"].tobytes(), f"half spmm {i} {red} {hv}"
            gv = oracle.spmm_value_bw(rowptr, col, mat, grad, red)
            assert sha(gv) == z[f"valuebw{i}_{red}"].tobytes(), f"value gradient {i} {red}"
        for red in ("max", "min"):
            for hv in (1, 0):
                o, arg = oracle.spmm_minmax(rowptr, col, val if hv else None, mat, red)
                assert sha(o) == z[f"minmax{i}_{red}_{hv}_out"].tobytes(), f"{red} {i} {hv}"
                assert sha(np.asarray(arg).astype(np.int64)) == z[f"minmax{i}_{red}_{hv}_arg"].tobytes(), f"{red} arg {i} {hv}"


def test_fp16_oracle_equals_torch_half_ops():
    """The fp16 restatement (quantize_activation_f16 / unpack_f16) against the same chain written with torch's
    half tensor ops on CPU, which round every Half (op) Half through fp32 like c10::Half in the reference's
    half kernels: statistics (ops.py:63, 39), codes (quantization_cuda_kernel.cu:89) and the reconstruction
    (quantization_cuda_kernel.cu:182), bit for bit."""
    import torch
    rng = np.random.default_rng(0)
    N, D = 3001, 37
    x = (rng.standard_normal((N, D)) * 3).astype(np.float16)
    u = rng.random((N, D), dtype=np.float32)
    for bits in (1, 2, 4, 8):
        p, s, m = oracle.quantize_activation_f16(x, u, bits)
        xt = torch.from_numpy(x)
        mn, mx = xt.min(1)[0], xt.max(1)[0]
        sc = (2 ** bits - 1) / (mx - mn)
        assert np.array_equal(sc.numpy().view(np.uint16), s.view(np.uint16))
        assert np.array_equal(mn.numpy().view(np.uint16), m.view(np.uint16))
        t = ((xt - mn[:, None]) * sc[:, None]).float() + torch.from_numpy(u)
        code = torch.clamp((t.double() - 0.5).float(), min=0).round().to(torch.int64).numpy()
        wpt = 8 // bits
        G = (N + wpt - 1) // wpt
        pad = np.zeros((G * wpt, D), np.int64)
        pad[:N] = code
        ref = np.zeros((G, D), np.int64)
        for i in range(wpt):
            ref |= pad[i::wpt] << (i * bits)
        assert np.array_equal((ref & 255).astype(np.uint8).ravel(), p)
        codes = np.stack([(p.reshape(G, D) >> (i * bits)) & ((1 << bits) - 1) for i in range(wpt)], 1)
        codes = codes.reshape(G * wpt, D)[:N]
        ref_un = torch.from_numpy(codes.astype(np.float32)).half() / sc[:, None] + mn[:, None]
        assert np.array_equal(ref_un.numpy().view(np.uint16), oracle.unpack_f16(p, s, m, N, D, bits).view(np.uint16))
