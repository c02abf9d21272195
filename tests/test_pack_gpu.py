"""GPU parity of pack / unpack / fused quantize_activation against the CPU oracle (bit-exact)."""
import numpy as np
import pytest
import torch

import oracle
from exact_b200 import config, dequantize_activation, quantize_activation
from exact_b200.cpp_extension import quantization as Q
from helpers import normal, relu_normal, uniform01

pytestmark = pytest.mark.gpu

SHAPES = [(4096, 128), (37, 13), (130, 602), (1001, 76), (513, 256), (64, 64), (77, 40), (9, 32), (250, 100),
          (33, 1), (64, 1024), (19, 2048), (8, 8), (1, 128), (7, 301)]
BITS = [1, 2, 4, 8]


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def u8(t):
    return t.cpu().numpy().view(np.uint8)


@pytest.mark.parametrize("bits", BITS)
@pytest.mark.parametrize("shape", SHAPES)
def test_fused_quantize_pack_supplied_noise(shape, bits):
    N, D = shape
    x, u = relu_normal(N, D, 11), uniform01((N, D), 12)
    packed, sb, mb, sf, mf = Q.quantize_pack(dev(x), bits, noise=dev(u), want_f32_stats=True)
    op, osb, omb, osf, omf = oracle.quantize_activation(x, u, bits)
    assert packed.numel() == op.size + 1
    assert np.array_equal(sf.cpu().numpy().view(np.int32), osf.view(np.int32))
    assert np.array_equal(mf.cpu().numpy(), omf)
    assert np.array_equal(sb.view(torch.int16).cpu().numpy().view(np.uint16), osb)
    assert np.array_equal(mb.view(torch.int16).cpu().numpy().view(np.uint16), omb)
    assert np.array_equal(u8(packed)[:-1], op)


@pytest.mark.parametrize("bits", BITS)
@pytest.mark.parametrize("shape", [(4096, 128), (37, 13), (130, 602), (513, 256)])
def test_fused_quantize_pack_philox(shape, bits):
    """Production noise: the kernel's Philox stream equals the oracle's restatement of it."""
    N, D = shape
    x = normal(N, D, 21)
    seed, offset = 0x1234567890ABCDEF, 77
    packed, sb, mb = Q.quantize_pack(dev(x), bits, seed=seed, offset=offset, row_offset=0)
    u = oracle.noise_b200(seed, offset, N, D)
    assert u.min() > 0 and u.max() < 1
    op, osb, omb, _, _ = oracle.quantize_activation(x, u, bits)
    assert np.array_equal(u8(packed)[:-1], op)
    assert np.array_equal(sb.view(torch.int16).cpu().numpy().view(np.uint16), osb)


def test_row_sharded_stream_equals_whole():
    """Shards of a multiple of 8 rows, keyed by their global row offset, concatenate to the stream of
    the unsharded call (what the multi-GPU row partition relies on)."""
    N, D, bits = 1000, 128, 2
    x = relu_normal(N, D, 31)
    whole, sb, mb = Q.quantize_pack(dev(x), bits, seed=5, offset=9, row_offset=0)
    cut = 496
    a, sa, ma = Q.quantize_pack(dev(x[:cut]), bits, seed=5, offset=9, row_offset=0)
    b, sb2, mb2 = Q.quantize_pack(dev(x[cut:]), bits, seed=5, offset=9, row_offset=cut)
    cat = np.concatenate([u8(a)[:-1], u8(b)[:-1]])
    assert np.array_equal(cat, u8(whole)[:-1])
    assert torch.equal(torch.cat([sa, sb2]), sb)


@pytest.mark.parametrize("bits", BITS)
@pytest.mark.parametrize("shape", [(4096, 128), (37, 13), (130, 602), (1001, 76)])
def test_pack_single_precision_reference_signature(shape, bits):
    """quantization.pack_single_precision(data, min, max, scale, bits, stochastic) with caller stats."""
    N, D = shape
    x, u = relu_normal(N, D, 41), uniform01((N, D), 42)
    xt = dev(x)
    mn, mx = torch.min(xt, 1)[0], torch.max(xt, 1)[0]
    scale = (2 ** bits - 1) / (mx - mn)
    packed = Q.pack_single_precision(xt, mn, mx, scale, bits, True, noise=dev(u))
    omn, omx, osc = oracle.row_stats(x, bits)
    assert np.array_equal(scale.cpu().numpy().view(np.int32), osc.view(np.int32))
    assert np.array_equal(u8(packed)[:-1], oracle.pack(x, omn, osc, u, bits))


@pytest.mark.parametrize("bits", BITS)
@pytest.mark.parametrize("shape", SHAPES)
@pytest.mark.parametrize("stats", ["bf16", "f32"])
def test_unpack(shape, bits, stats):
    N, D = shape
    x, u = relu_normal(N, D, 51), uniform01((N, D), 52)
    op, osb, omb, osf, omf = oracle.quantize_activation(x, u, bits)
    pk = torch.from_numpy(np.concatenate([op, np.zeros(1, np.uint8)]).view(np.int8)).cuda()
    if stats == "bf16":
        s = torch.from_numpy(osb.view(np.int16)).cuda().view(torch.bfloat16)
        m = torch.from_numpy(omb.view(np.int16)).cuda().view(torch.bfloat16)
        ref = oracle.dequantize_activation(op, osb, omb, N, D, bits)
    else:
        s, m = dev(osf), dev(omf)
        ref = oracle.unpack(op, osf, omf, N, D, bits)
    out = Q.unpack_single_precision(pk, bits, s, m, N, D)
    assert np.array_equal(out.cpu().numpy(), ref)  # bit-exact, tighter than the 1e-6 relative asked for


def test_bf16_input_is_widened_then_quantised():
    N, D, bits = 257, 128, 2
    xb = torch.from_numpy(relu_normal(N, D, 61)).to(torch.bfloat16)
    u = uniform01((N, D), 62)
    packed, sb, mb = Q.quantize_pack(xb.cuda(), bits, noise=dev(u))
    op, osb, omb, _, _ = oracle.quantize_activation(xb.float().numpy(), u, bits)
    assert np.array_equal(u8(packed)[:-1], op)
    assert np.array_equal(sb.view(torch.int16).cpu().numpy().view(np.uint16), osb)


def test_edge_cases_constant_rows_nan_and_empty():
    x = relu_normal(16, 32, 71)
    x[3] = 0.5          # constant row: scale = inf, codes 0
    x[5, 7] = np.nan    # NaN row: stats NaN, codes 0
    u = uniform01((16, 32), 72)
    packed, sb, mb, sf, mf = Q.quantize_pack(dev(x), 2, noise=dev(u), want_f32_stats=True)
    op, osb, omb, osf, omf = oracle.quantize_activation(x, u, 2)
    assert np.array_equal(u8(packed)[:-1], op)
    assert np.array_equal(sf.cpu().numpy().view(np.int32)[[0, 3]], osf.view(np.int32)[[0, 3]])
    assert np.isnan(sf[5].item()) and np.isnan(mf[5].item()) and np.isinf(sf[3].item())
    e = torch.empty(0, 128, device="cuda")
    pk, s, m = Q.quantize_pack(e, 2)
    assert pk.numel() == 1 and s.numel() == 0


def test_no_upper_clamp_is_reproduced():
    x = np.zeros((4, 8), np.float32)
    x[0, :] = np.linspace(0, 3.6, 8)
    mn = np.zeros(4, np.float32)
    mx = np.full(4, 3.6, np.float32)
    sc = np.ones(4, np.float32)
    u = np.full((4, 8), 0.5, np.float32)
    packed = Q.pack_single_precision(dev(x), dev(mn), dev(mx), dev(sc), 2, True, noise=dev(u))
    ref = oracle.pack(x, mn, sc, u, 2)
    assert ref[7] == 4
    assert np.array_equal(u8(packed)[:-1], ref)


def test_public_api_round_trip_config1():
    """Benchmark configuration 1, first half: 4096 x 128, INT2, supplied noise, through the reference's API."""
    config.activation_compression_bits = [2]
    config.compress_activation = True
    x, u = relu_normal(4096, 128, 0), uniform01((4096, 128), 1)
    q = quantize_activation(dev(x), None, noise=dev(u))
    assert q[1] == 2 and q[2].dtype == torch.bfloat16 and q[0].dtype == torch.int8
    xh = dequantize_activation(q, (4096, 128))
    op, osb, omb, _, _ = oracle.quantize_activation(x, u, 2)
    assert np.array_equal(u8(q[0])[:-1], op)
    assert np.array_equal(xh.cpu().numpy(), oracle.dequantize_activation(op, osb, omb, 4096, 128, 2))


def test_unbiasedness_of_stochastic_rounding():
    """The statistic the reference prints (test/test_op.py:322-330): the mean of many quantised copies
    approaches the input."""
    N, D = 256, 128
    x = relu_normal(N, D, 81)
    xt = dev(x)
    acc = torch.zeros_like(xt)
    reps = 200
    for i in range(reps):
        pk, sb, mb, sf, mf = Q.quantize_pack(xt, 2, seed=3, offset=i, want_f32_stats=True)
        acc += Q.unpack_single_precision(pk, 2, sf, mf, N, D)
    err = (acc / reps - xt).abs().max().item()
    step = float((x.max(1) - x.min(1)).max() / 3)
    assert err < 0.15 * step


def test_full_size_round_trip_properties():
    """At benchmark size (10^6 x 128): decode(encode(x)) stays within one quantisation step, codes use
    the full range, and a checksum of the packed stream is reproducible for the same (seed, offset)."""
    N, D, bits = 1_000_000, 128, 2
    g = torch.Generator(device="cuda").manual_seed(5)
    x = torch.randn(N, D, device="cuda", generator=g).relu_()
    pk, sb, mb, sf, mf = Q.quantize_pack(x, bits, seed=1, offset=2, want_f32_stats=True)
    pk2, _, _ = Q.quantize_pack(x, bits, seed=1, offset=2)
    assert torch.equal(pk[:-1], pk2[:-1])
    xh = Q.unpack_single_precision(pk, bits, sf, mf, N, D)
    step = (x.max(1)[0] - x.min(1)[0]) / 3
    assert bool(((xh - x).abs() <= step[:, None] * 1.001 + 1e-6).all())
    assert torch.equal(mf, x.min(1)[0])


@pytest.mark.parametrize("bits", BITS)
def test_unpack_division_is_ieee_for_any_scale(bits):
    """The dequantise uses a reciprocal-based quotient for ordinary scales and the division sequence
    otherwise; both must equal the oracle's IEEE division: scales across the whole float range,
    infinities (constant rows), denormals, negative and NaN scales."""
    N, D = 4096, 64
    rng = np.random.default_rng(91)
    wpt = 8 // bits
    packed = rng.integers(0, 256, size=(N // wpt) * D, dtype=np.uint8)
    bits32 = rng.integers(0, 2 ** 32, size=N, dtype=np.uint64).astype(np.uint32)
    scale = bits32.view(np.float32).copy()           # every exponent, both signs, some NaN/inf
    scale[:64] = np.float32(np.inf)
    scale[64:128] = np.float32(1e-41)                # denormal
    scale[128:2048] = rng.uniform(0.01, 300.0, 1920).astype(np.float32)   # the ordinary range
    mn = rng.standard_normal(N).astype(np.float32)
    ref = oracle.unpack(packed, scale, mn, N, D, bits)
    pk = torch.from_numpy(np.concatenate([packed, np.zeros(1, np.uint8)]).view(np.int8)).cuda()
    out = Q.unpack_single_precision(pk, bits, dev(scale), dev(mn), N, D).cpu().numpy()
    assert np.array_equal(out.view(np.uint32)[~np.isnan(ref)], ref.view(np.uint32)[~np.isnan(ref)])
    assert np.array_equal(np.isnan(out), np.isnan(ref))


@pytest.mark.parametrize("bits", BITS)
@pytest.mark.parametrize("D", [128, 602])
def test_philox_path_with_constant_inf_and_nan_rows(bits, D):
    """Full tiles with Philox noise take a conversion-free rounding path unless a row of the tile is
    constant (scale = inf), or holds an infinity (scale = 0) or a NaN; those tiles must still equal the
    oracle bit for bit."""
    N = 4096
    x = relu_normal(N, D, 93)
    x[8:16] = 0.0                 # a whole tile of constant rows (all-zero activations)
    x[37] = 1.25                  # a constant row inside an otherwise ordinary tile
    x[100, 5] = np.inf
    x[203, 7] = -np.inf
    x[300, 9] = np.nan
    x[401] = np.float32(3e38); x[401, 0] = np.float32(-3e38)   # range overflows to inf
    x[500, :] = np.float32(1e-39); x[500, 3] = np.float32(2e-39)  # denormal range -> scale = inf
    seed, offset = 11, 5
    packed, sb, mb, sf, mf = Q.quantize_pack(dev(x), bits, seed=seed, offset=offset, row_offset=0, want_f32_stats=True)
    u = oracle.noise_b200(seed, offset, N, D)
    op, osb, omb, osf, omf = oracle.quantize_activation(x, u, bits)
    assert np.array_equal(sf.cpu().numpy().view(np.uint32)[~np.isnan(osf)], osf.view(np.uint32)[~np.isnan(osf)])
    assert np.array_equal(np.isnan(sf.cpu().numpy()), np.isnan(osf))
    assert np.array_equal(u8(packed)[:-1], op)


def test_swap_round_trip_equals_on_device_result():
    """config.swap (utils.py:31-34, ops.py:41-42, 50-51): the packed stream is parked in pinned host memory and
    brought back for backward; the dequantised activation equals the one that never left the device."""
    from exact_b200 import dequantize_activation, quantize_activation
    config.compress_activation, config.kept_frac, config.activation_compression_bits = True, 1.0, [2]
    x = torch.from_numpy(relu_normal(3001, 96, 17)).cuda()
    u = torch.from_numpy(uniform01((3001, 96), 18)).cuda()
    try:
        config.swap = False
        q_dev = quantize_activation(x, None, noise=u)
        ref = dequantize_activation(q_dev, x.shape)
        config.swap = True
        q_host = quantize_activation(x, None, noise=u)
        assert not q_host[0].is_cuda and q_host[0].is_pinned()
        assert torch.equal(q_host[0][:-1], q_dev[0][:-1].cpu())
        back = dequantize_activation(q_host, x.shape)
        assert back.is_cuda and torch.equal(back, ref)
        # a layer's backward through the swapped copy
        lin = torch.nn.Linear(96, 8).cuda()
        from exact_b200.ops import qlinear
        xa = x.clone().requires_grad_()
        config.manual_seed(5)
        qlinear.apply(xa, lin.weight, lin.bias).sum().backward()
        g_swap, w_swap = xa.grad.clone(), lin.weight.grad.clone()
        lin.weight.grad = None
        config.swap = False
        xb = x.clone().requires_grad_()
        config.manual_seed(5)
        qlinear.apply(xb, lin.weight, lin.bias).sum().backward()
        assert torch.equal(g_swap, xb.grad) and torch.equal(w_swap, lin.weight.grad)
    finally:
        config.swap = False
