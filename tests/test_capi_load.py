"""CPU checks of the C-ABI library: it loads, exports every symbol include/*.h declares, and its
argument validation works without touching a GPU."""
import ctypes
import glob
import os
import re

from exact_b200 import _build, _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    names = []
    for h in glob.glob(os.path.join(ROOT, "include", "*.h")):
        src = open(h).read()
        names += re.findall(r"EXACT_API\s+[\w\s\*]+?\b(exact_\w+)\s*\(", src)
    return sorted(set(names))


def test_header_symbols_are_exported():
    names = declared_symbols()
    assert len(names) >= 12
    lib = ctypes.CDLL(_build.LIB)
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/ but not exported"


def test_bindings_cover_the_header():
    assert sorted(_lib.SIGNATURES) == declared_symbols()


def test_host_only_entry_points():
    lib = _lib.load()
    assert lib.exact_version() >= 100
    assert lib.exact_packed_bytes(4096, 128, 2) == 131072
    assert lib.exact_packed_bytes(169343, 256, 2) == 42336 * 256
    assert lib.exact_packed_bytes(5, 3, 8) == 15
    assert lib.exact_packed_bytes(5, 3, 3) == -1
    assert lib.exact_mask_words(0) == 0 and lib.exact_mask_words(129) == 8 and lib.exact_mask_words(257) == 16


def test_bad_arguments_are_rejected_before_any_launch():
    lib = _lib.load()
    rc = lib.exact_quantize_pack(None, 0, 8, 8, 3, None, 0, 0, 0, None, None, None, None, None, None)
    assert rc == 1 and b"bits" in lib.exact_last_error()
    rc = lib.exact_quantize_pack(None, 0, 8, 8, 2, None, 0, 0, 4, None, None, None, None, None, None)
    assert rc == 1 and b"row_offset" in lib.exact_last_error()
    rc = lib.exact_quantize_pack(None, 0, 8, 8, 2, None, 0, 0, 0, None, None, None, None, None, None)
    assert rc == 1 and b"null" in lib.exact_last_error()
    rc = lib.exact_spmm(None, None, 2, None, None, 4, 4, 0, None, None)
    assert rc == 1 and b"idx_bytes" in lib.exact_last_error()
    # empty inputs are a no-op, as torch.empty-shaped calls are in the reference
    assert lib.exact_quantize_pack(None, 0, 0, 128, 2, None, 0, 0, 0, None, None, None, None, None, None) == 0


def test_new_entry_points_reject_bad_arguments_without_a_gpu():
    lib = _lib.load()
    assert lib.exact_linear_workspace_bytes(256, 256, 0) == 256 + 2 * 256 * 256 * 4
    assert lib.exact_linear_workspace_bytes(47, 100, 256) == 256 + 2 * 48 * (128 + 256) * 4
    # N wider than one MMA tile and rows of A that are not 16-byte aligned are "unsupported" (code 3): the caller
    # keeps its library GEMM; a second operand pair needs all three of A2, B2, K2
    one = ctypes.c_void_p(16)
    rc = lib.exact_linear_forward(one, 8, 8, 8, one, 8, None, 0, 0, None, 0, 300, None, 0, one, one, 300, None)
    assert rc == 3 and b"256" in lib.exact_last_error()
    rc = lib.exact_linear_forward(one, 8, 6, 6, one, 6, None, 0, 0, None, 0, 8, None, 0, one, one, 8, None)
    assert rc == 3 and b"aligned" in lib.exact_last_error()
    rc = lib.exact_linear_forward(one, 8, 8, 8, one, 8, one, 0, 0, None, 0, 8, None, 0, one, one, 8, None)
    assert rc == 1
    assert lib.exact_linear_forward(None, 0, 8, 8, None, 8, None, 0, 0, None, 0, 8, None, 0, None, None, 8, None) == 0
    rc = lib.exact_rows_mask_count(one, 4, 48, 48, one, one, None)
    assert rc == 1 and b"multiple of 32" in lib.exact_last_error()
    rc = lib.exact_rows_expand(one, one, one, 4, 64, 0, 5, 64, one, 64, None)
    assert rc == 1
    assert lib.exact_rows_compact_write(None, 0, 64, 64, None, None, None) == 0


def test_dense_layer_host_logic_on_cpu():
    """Off the GPU (or below the row threshold, or with the switch off) the wrappers are the library ops."""
    import torch
    from exact_b200.cpp_extension import backward_func as B
    g = torch.Generator().manual_seed(0)
    a, w, b = torch.randn(50, 12, generator=g), torch.randn(7, 12, generator=g), torch.randn(7, generator=g)
    a2, w2 = torch.randn(50, 5, generator=g), torch.randn(7, 5, generator=g)
    assert torch.equal(B.linear_forward(a, w, b), torch.nn.functional.linear(a, w, b))
    ref = torch.nn.functional.linear(a, w, b) + a2 @ w2.t()
    assert torch.allclose(B.linear_forward(a, w, b, a2=a2, weight2=w2), ref, atol=1e-6)
    out = torch.ones(50, 7)
    assert torch.allclose(B.linear_forward(a, w, None, out=out, accumulate=True), 1 + a @ w.t(), atol=1e-6)
    gi, gw, gb = B.linear_backward(torch.randn(50, 7, generator=g), a, w, b, need_grad_input=False)
    assert gi is None and gw.shape == (7, 12) and gb.shape == (7,)
    # rows whose pitch is not a multiple of 16 bytes are copied into padded rows, values unchanged
    v = torch.randn(9, 47, generator=g)
    p = B._rows16(v)
    assert p.shape == v.shape and torch.equal(p, v) and p.stride(0) == 48
    big = torch.randn(70000, 6, generator=g)
    x = torch.randn(70000, 3, generator=g)
    assert torch.allclose(B.rows_reduce_mm(big, x), big.t() @ x, rtol=1e-4, atol=1e-3)


def test_argument_checks_added_later_reject_before_any_launch():
    lib = _lib.load()
    one, odd = ctypes.c_void_p(256), ctypes.c_void_p(258)
    # the fused projection + pack stores 32-bit words of packed bytes when k % 4 == 0: an unaligned `packed` is
    # an argument error (code 1), not a misaligned store on the device
    rc = lib.exact_rp_quantize_pack(one, 128, 64, one, 8, 2, 0, 0, 0, one, odd, one, one, None, None)
    assert rc == 1 and b"4-byte aligned" in lib.exact_last_error()
    # the static-scratch entry compares n_items * K with its limit without overflowing int64
    big = 1 << 62
    rc = lib.exact_spmm_split_static(one, one, 4, None, one, 8, 256, 0, 256, one, one, one, None, big, one, one, 1, one,
                                     None)
    assert rc == 1 and b"built-in scratch" in lib.exact_last_error()
    # compact rows: at most 256 columns, 1..8 aligned destinations
    assert lib.exact_crows_slot_bytes(256) == 16 + 256 + 1024 and lib.exact_crows_slot_bytes(100) == 16 + 112 + 400
    assert lib.exact_crows_slot_bytes(257) == -1
    dst = (ctypes.c_void_p * 1)(odd.value)
    rc = lib.exact_crows_pack(one, 4, 64, 64, None, 0, dst, 1, None, None)
    assert rc == 1 and b"aligned" in lib.exact_last_error()
    rc = lib.exact_crows_pack(one, 4, 300, 300, None, 0, dst, 1, None, None)
    assert rc == 1 and b"256" in lib.exact_last_error()
    rc = lib.exact_crows_pack(one, 4, 64, 64, None, 0, dst, 9, None, None)
    assert rc == 1
    rc = lib.exact_spmm(one, one, 4, None, one, (1 << 32) + 8, 4, 0, one, None)
    assert rc == 1 and b"2^32" in lib.exact_last_error()


def test_entry_points_added_for_routing_batch_norm_and_fp16_reject_bad_arguments():
    lib = _lib.load()
    one = ctypes.c_void_p(256)
    dst = (ctypes.c_void_p * 2)(256, 512)
    # routed SpMM: the destinations must hold all rows, the columns must fit the row pitch
    rc = lib.exact_spmm_split_routed(one, one, 4, None, one, 100, 32, 0, 0, None, None, None, None, 0, None, None, 0, None,
                                     None, 40, 0, 32, dst, 2, None)
    assert rc == 1 and b"do not hold" in lib.exact_last_error()
    rc = lib.exact_spmm_split_routed(one, one, 4, None, one, 100, 32, 0, 0, None, None, None, None, 0, None, None, 0, None,
                                     None, 50, 16, 32, dst, 2, None)
    assert rc == 1 and b"row pitch" in lib.exact_last_error()
    rc = lib.exact_spmm_split_routed(one, one, 4, None, one, 100, 32, 0, 0, None, None, None, None, 0, None, None, 0, None,
                                     None, 50, 0, 32, dst, 9, None)
    assert rc == 1
    # batch-norm backward from the packed input: D % 4 != 0 is "unsupported" (the caller unpacks), a short
    # workspace an argument error
    assert lib.exact_bn_backward_from_packed(one, 8, 13, one, 2, one, one, None, one, one, 1, one, 1 << 20, one, one, one,
                                             None) == 3
    rc = lib.exact_bn_backward_from_packed(one, 8, 16, one, 2, one, one, None, one, one, 1, one, 16, one, one, one, None)
    assert rc == 1 and b"workspace" in lib.exact_last_error()
    # fp16 entry points
    assert lib.exact_quantize_pack_f16(one, 8, 16, 3, None, 0, 0, 0, one, one, one, None) == 1
    assert lib.exact_quantize_pack_f16(one, 8, 16, 2, None, 0, 0, 4, one, one, one, None) == 1   # row_offset % 8
    assert lib.exact_unpack_single_precision_f16(None, 2, one, one, 8, 16, one, None) == 1
    assert lib.exact_act_quantized_forward_f16(7, one, 8, 0.0, None, 0, 0, 0, one, one, None) == 1
    assert lib.exact_act_quantized_forward_f16(1, one, 8, 1.5, None, 0, 0, 0, one, one, None) == 1   # p > 1
    assert lib.exact_spmm_f16(one, one, 2, None, one, 8, 16, 0, one, None) == 1


def test_device_of_a_call_comes_from_its_tensors():
    """invoke() launches on the device its tensor arguments live on and refuses mixed devices."""
    import pytest
    assert _lib.resolve_device({1}, 0) == 1
    assert _lib.resolve_device(set(), 3) == 3
    with pytest.raises(_lib.ExactB200Error, match="different CUDA devices"):
        _lib.resolve_device({0, 1}, 0)


def test_status_word_turns_into_an_exception():
    import pytest
    _lib.raise_for_status(0)
    with pytest.raises(_lib.ExactB200Error, match="exact_rp_quantize_pack"):
        _lib.raise_for_status(1)
    with pytest.raises(_lib.ExactB200Error, match="exact_unpack_dequant_rp, exact_linear_forward"):
        _lib.raise_for_status(6)


def test_benchmark_knobs_follow_the_reference_driver():
    """--n_bits / --kept_frac / --act_fp as mem_speed_bench/arxiv/train_full_batch.py:120-137 maps them."""
    import argparse
    import importlib.util
    import os
    from exact_b200 import config, graphs
    spec = importlib.util.spec_from_file_location("bench", os.path.join(ROOT, "bench.py"))
    bench = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(bench)
    ns = lambda **kw: argparse.Namespace(**dict(dict(n_bits=None, kept_frac=None, act_fp=False, no_compress=False), **kw))
    try:
        c = bench.apply_knobs(graphs.CONFIGS["cfg3"], ns())
        assert config.compress_activation and config.activation_compression_bits == [2] and config.kept_frac == 0.125
        assert c["use_qmodule"] and "int2_kf0.125" in bench.workload_name(c, 5)
        c = bench.apply_knobs(graphs.CONFIGS["cfg3"], ns(n_bits=4, kept_frac=0.5))
        assert config.activation_compression_bits == [4] and config.kept_frac == 0.5 and c["use_qmodule"]
        # fp32 activations with a projection: the quantised modules stay, compression is off, the projection applies
        c = bench.apply_knobs(graphs.CONFIGS["cfg3"], ns(act_fp=True))
        assert not config.compress_activation and config.kept_frac == 0.125 and c["use_qmodule"]
        assert "fp32act_kf0.125" in bench.workload_name(c, 5)
        # fp32 activations without projection: the unwrapped model
        c = bench.apply_knobs(graphs.CONFIGS["cfg2"], ns(act_fp=True))
        assert not config.compress_activation and config.kept_frac == 1.0 and not c["use_qmodule"]
    finally:
        config.compress_activation, config.activation_compression_bits, config.kept_frac = True, [2], 1.0


def test_aggregation_mode_follows_the_world_size_unless_forced():
    from exact_b200 import config
    from exact_b200.dist import column_split_active, shard_rows
    old = config.column_split_aggregation
    try:
        config.column_split_aggregation = None
        assert [column_split_active(w) for w in (1, 2, 4, 8, 16)] == [False, False, False, True, True]
        config.column_split_aggregation = True
        assert column_split_active(2)
        config.column_split_aggregation = False
        assert not column_split_active(8)
    finally:
        config.column_split_aggregation = old
    # shards are multiples of 8 rows (packed streams of the shards concatenate to the single-GPU stream)
    assert shard_rows(2449029, 8) % 8 == 0 and shard_rows(2449029, 8) * 8 >= 2449029
    assert shard_rows(10, 4) == 8
