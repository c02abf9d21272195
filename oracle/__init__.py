"""CPU oracle for the EXACT activation-compression hot path -- TEST INFRASTRUCTURE ONLY.

numpy-facing wrappers around oracle/exact_oracle.c (a C restatement of the reference's CUDA kernels
and of the torch glue in exact/exact/ops.py).  Only tests, the smoke check and the benchmark's CPU
baseline may import this package; the product (exact_b200) never does.

Parity pin: see the header of exact_oracle.c.
"""
import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SRC = os.path.join(_HERE, "exact_oracle.c")
_SO = os.path.join(_HERE, "liboracle.so")
_lib = None


def build(force=False):
    """Compile exact_oracle.c with gcc (no fused-multiply-add contraction, OpenMP)."""
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(_SRC):
        cmd = ["gcc", "-O2", "-ffp-contract=off", "-fopenmp", "-shared", "-fPIC", "-fvisibility=hidden",
               _SRC, "-o", _SO, "-lm"]
        subprocess.run(cmd, check=True)
    return _SO


def lib():
    global _lib
    if _lib is None:
        build()
        _lib = ctypes.CDLL(_SO)
    return _lib


def _p(a):
    return None if a is None else a.ctypes.data_as(ctypes.c_void_p)


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


i64 = ctypes.c_int64
u64 = ctypes.c_uint64
cint = ctypes.c_int


def f32_to_bf16(x):
    x = _f32(x)
    out = np.empty(x.shape, np.uint16)
    lib().orc_f32_to_bf16(_p(x), i64(x.size), _p(out))
    return out


def bf16_to_f32(x):
    x = np.ascontiguousarray(x, dtype=np.uint16)
    out = np.empty(x.shape, np.float32)
    lib().orc_bf16_to_f32(_p(x), i64(x.size), _p(out))
    return out


def row_stats(x, bits):
    """-> (mn, mx, scale), fp32 [N].  ops.py:61-66, ops.py:39."""
    x = _f32(x)
    N, D = x.shape
    mn, mx, sc = (np.empty(N, np.float32) for _ in range(3))
    lib().orc_row_stats(_p(x), i64(N), i64(D), cint(bits), _p(mn), _p(mx), _p(sc))
    return mn, mx, sc


def packed_nbytes(N, D, bits):
    wpt = 8 // bits
    return ((N + wpt - 1) // wpt) * D


def pack(x, mn, scale, noise, bits, use_fma=True):
    """pack_single_precision (quantization_cuda_kernel.cu:73-93) -> uint8 [ceil(N/wpt)*D]."""
    x, mn, scale, noise = _f32(x), _f32(mn), _f32(scale), _f32(noise)
    N, D = x.shape
    out = np.empty(packed_nbytes(N, D, bits), np.uint8)
    lib().orc_pack(_p(x), _p(mn), _p(scale), _p(noise), i64(N), i64(D), cint(bits), cint(int(use_fma)),
                   _p(out))
    return out


def unpack(packed, scale, mn, N, D, bits):
    """unpack_single_precision (quantization_cuda_kernel.cu:167-184) -> fp32 [N, D]."""
    packed = np.ascontiguousarray(packed).view(np.uint8)
    scale, mn = _f32(scale), _f32(mn)
    out = np.empty((N, D), np.float32)
    lib().orc_unpack(_p(packed), _p(scale), _p(mn), i64(N), i64(D), cint(bits), _p(out))
    return out


def quantize_activation(x, noise, bits, use_fma=True):
    """ops.py:69-83 for fp32 input -> (packed u8, scale bf16-bits u16, min bf16-bits u16, scale f32, min f32)."""
    x, noise = _f32(x), _f32(noise)
    N, D = x.shape
    packed = np.empty(packed_nbytes(N, D, bits), np.uint8)
    sb, mb = np.empty(N, np.uint16), np.empty(N, np.uint16)
    sf, mf = np.empty(N, np.float32), np.empty(N, np.float32)
    lib().orc_quantize_activation(_p(x), _p(noise), i64(N), i64(D), cint(bits), cint(int(use_fma)),
                                  _p(packed), _p(sb), _p(mb), _p(sf), _p(mf))
    return packed, sb, mb, sf, mf


def dequantize_activation(packed, scale_bf16, min_bf16, N, D, bits):
    """ops.py:86-98 -> fp32 [N, D]."""
    packed = np.ascontiguousarray(packed).view(np.uint8)
    sb = np.ascontiguousarray(scale_bf16, dtype=np.uint16)
    mb = np.ascontiguousarray(min_bf16, dtype=np.uint16)
    out = np.empty((N, D), np.float32)
    lib().orc_dequantize_activation(_p(packed), _p(sb), _p(mb), i64(N), i64(D), cint(bits), _p(out))
    return out


def philox4x32_10(ctr, key):
    c = np.asarray(ctr, np.uint32)
    k = np.asarray(key, np.uint32)
    out = np.empty(4, np.uint32)
    lib().orc_philox4x32_10(_p(c), _p(k), _p(out))
    return out


def noise_reference_pack(seed, offset, N, D, bits):
    """The U(0,1] noise the reference's pack kernel draws for (seed, philox offset)."""
    out = np.zeros((N, D), np.float32)
    lib().orc_noise_reference_pack(u64(seed), u64(offset), i64(N), i64(D), cint(bits), _p(out))
    return out


def noise_b200(seed, offset, N, D, row_offset=0):
    """The production stochastic-rounding noise of the B200 library for (seed, offset)."""
    out = np.zeros((N, D), np.float32)
    lib().orc_noise_b200(u64(seed), u64(offset), i64(row_offset), i64(N), i64(D), _p(out))
    return out


def noise_b200_rows(seed, offset, N, k, row_offset=0):
    """The stochastic-rounding noise of the B200 library's fused projection+pack kernel."""
    out = np.zeros((N, k), np.float32)
    lib().orc_noise_b200_rows(u64(seed), u64(offset), i64(row_offset), i64(N), i64(k), _p(out))
    return out


def uniform_b200(seed, offset, n):
    """The production dropout uniforms of the B200 library for (seed, offset)."""
    out = np.zeros(n, np.float32)
    lib().orc_uniform_b200(u64(seed), u64(offset), i64(n), _p(out))
    return out


def rademacher(seed, offset, D, k):
    """The seeded +-1/sqrt(k) matrix [D, k] of the B200 library's input2rp."""
    out = np.empty((D, k), np.float32)
    lib().orc_rademacher(u64(seed), u64(offset), i64(D), i64(k), _p(out))
    return out


def relu_fw(x):
    x = _f32(x)
    out = np.empty_like(x)
    keep = np.empty(x.shape, np.uint8)
    lib().orc_relu_fw(_p(x), i64(x.size), _p(out), _p(keep))
    return out, keep


def mask_bw(g, keep):
    g = _f32(g)
    keep = np.ascontiguousarray(keep, dtype=np.uint8)
    out = np.empty_like(g)
    lib().orc_mask_bw(_p(g), _p(keep), i64(g.size), _p(out))
    return out


def dropout_fw(x, u, p):
    x, u = _f32(x), _f32(u)
    out = np.empty_like(x)
    keep = np.empty(x.shape, np.uint8)
    lib().orc_dropout_fw(_p(x), _p(u), ctypes.c_float(p), i64(x.size), _p(out), _p(keep))
    return out, keep


def dropout_bw(g, keep, p):
    g = _f32(g)
    keep = np.ascontiguousarray(keep, dtype=np.uint8)
    out = np.empty_like(g)
    lib().orc_dropout_bw(_p(g), _p(keep), ctypes.c_float(p), i64(g.size), _p(out))
    return out


def input2rp(x, R):
    x, R = _f32(x), _f32(R)
    N, D = x.shape
    k = R.shape[1]
    out = np.empty((N, k), np.float32)
    lib().orc_input2rp(_p(x), _p(R), i64(N), i64(D), i64(k), _p(out))
    return out


def rp2input(xq, R):
    xq, R = _f32(xq), _f32(R)
    N, k = xq.shape
    D = R.shape[0]
    out = np.empty((N, D), np.float32)
    lib().orc_rp2input(_p(xq), _p(R), i64(N), i64(D), i64(k), _p(out))
    return out


def spmm(rowptr, col, val, mat, reduce="sum"):
    """CSR x dense, reduce in {'sum','mean'} (spmm_cuda.cu:54-103, reducer.cuh:55-84)."""
    rowptr = np.ascontiguousarray(rowptr, dtype=np.int64)
    col = np.ascontiguousarray(col, dtype=np.int64)
    val = None if val is None else _f32(val)
    mat = _f32(mat)
    M = rowptr.size - 1
    K = mat.shape[1]
    out = np.empty((M, K), np.float32)
    lib().orc_spmm(_p(rowptr), _p(col), _p(val), _p(mat), i64(M), i64(K),
                   cint({"sum": 0, "mean": 1}[reduce]), _p(out))
    return out


def spmm_bw_mat(rowptr, col, val, grad_out, n_cols, reduce="sum"):
    """Gradient wrt the dense operand (spmm.cc:57-79 sum, 115-139 mean): SpMM over the transposed
    structure (colptr, row[csr2csc], weights[csr2csc]) with reduce='sum'."""
    rowptr = np.asarray(rowptr, np.int64)
    col = np.asarray(col, np.int64)
    M = rowptr.size - 1
    nnz = col.size
    row = np.repeat(np.arange(M, dtype=np.int64), np.diff(rowptr))
    perm = np.argsort(col * M + row, kind="stable")  # csr2csc
    colptr = np.zeros(n_cols + 1, np.int64)
    np.cumsum(np.bincount(col, minlength=n_cols), out=colptr[1:])
    row_t = row[perm]
    if reduce == "mean":
        cnt = np.maximum(np.diff(rowptr)[row_t].astype(np.float32), np.float32(1))
        if val is not None:
            w = _f32(val)[perm] / cnt
        else:
            w = np.float32(1) / cnt  # torch pow_(-1) on fp32 == IEEE reciprocal
    else:
        w = None if val is None else _f32(val)[perm]
    assert nnz == perm.size
    return spmm(colptr, row_t, w, grad_out, "sum")


def spmm_value_bw(rowptr, col, mat, grad, reduce="sum"):
    """Gradient wrt the edge values (spmm_cuda.cu:172-209): [nnz] fp32."""
    rowptr = np.ascontiguousarray(rowptr, np.int64)
    col = np.ascontiguousarray(col, np.int64)
    row = np.repeat(np.arange(rowptr.size - 1, dtype=np.int64), np.diff(rowptr))
    mat, grad = _f32(mat), _f32(grad)
    out = np.zeros(col.size, np.float32)
    lib().orc_spmm_value_bw(_p(row), _p(rowptr), _p(col), _p(mat), _p(grad), i64(col.size), i64(mat.shape[1]),
                            ctypes.c_int(1 if reduce == "mean" else 0), _p(out))
    return out


def spmm_minmax(rowptr, col, val, mat, reduce):
    """max / min aggregation -> (out [M, K] fp32, arg_out [M, K] int64; nnz where a row has no edge)."""
    rowptr = np.ascontiguousarray(rowptr, np.int64)
    col = np.ascontiguousarray(col, np.int64)
    mat = _f32(mat)
    M, K = rowptr.size - 1, mat.shape[1]
    v = None if val is None else _f32(val)
    out = np.zeros((M, K), np.float32)
    arg = np.zeros((M, K), np.int64)
    lib().orc_spmm_minmax(_p(rowptr), _p(col), _p(v) if v is not None else None, _p(mat), i64(M), i64(K), i64(col.size),
                          ctypes.c_int(1 if reduce == "max" else 0), _p(out), _p(arg))
    return out, arg


def rows_compact(x):
    """Zero-compacted rows of x [n, K] fp32, K % 32 == 0 (the exchange format of the row-sharded
    aggregation; no counterpart in the reference): mask uint32 [n, K/32] (bit c % 32 of word c / 32 set
    when any bit of element c is set), rowoff int64 [n + 1], vals fp32 (kept elements, row-major)."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    n, K = x.shape
    keep = x.view(np.uint32) != 0
    weights = (np.uint64(1) << np.arange(32, dtype=np.uint64))
    mask = (keep.reshape(n, K // 32, 32).astype(np.uint64) * weights).sum(-1).astype(np.uint32)
    rowoff = np.zeros(n + 1, dtype=np.int64)
    np.cumsum(keep.sum(1), out=rowoff[1:])
    return mask, rowoff, x[keep]


def rows_expand(mask, rowoff, vals, K):
    """Inverse of rows_compact."""
    n = mask.shape[0]
    keep = ((mask[:, :, None] >> np.arange(32, dtype=np.uint32)) & 1).astype(bool).reshape(n, K)
    out = np.zeros((n, K), dtype=np.float32)
    out[keep] = vals[:rowoff[n]]
    return out


def crows_slot_bytes(K):
    """Bytes of one compact-row slot: 16-byte header, column bytes padded to 16, K fp32 values."""
    return 16 + (K + 15) // 16 * 16 + 4 * K


def crows_pack(x, rowscale=None):
    """Compact rows of x [n, K] fp32 (K <= 256), optionally x * rowscale[:, None] in fp32 first (no counterpart
    in the reference): a zero-filled uint8 buffer [n, slot] with, per row, uint32 count at +0, the kept columns
    (any of the 32 bits set) ascending at +16 and their values at +16 + pad16(K)."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    if rowscale is not None:
        x = (x * np.asarray(rowscale, dtype=np.float32).reshape(-1, 1)).astype(np.float32)
    n, K = x.shape
    slot = crows_slot_bytes(K)
    voff = 16 + (K + 15) // 16 * 16
    buf = np.zeros((n, slot), dtype=np.uint8)
    bits = x.view(np.uint32)
    for r in range(n):
        cols = np.nonzero(bits[r])[0]
        buf[r, 0:4] = np.array([cols.size], dtype=np.uint32).view(np.uint8)
        buf[r, 16:16 + cols.size] = cols.astype(np.uint8)
        buf[r, voff:voff + 4 * cols.size] = bits[r, cols].view(np.uint8)
    return buf


def crows_used_mask(buf, K):
    """Boolean [n, slot]: the bytes of each slot that crows_pack defines (header word, used columns and values)."""
    n, slot = buf.shape
    voff = 16 + (K + 15) // 16 * 16
    cnt = buf[:, 0:4].copy().view(np.uint32).reshape(n).astype(np.int64)
    pos = np.arange(slot)[None, :]
    return (pos < 4) | ((pos >= 16) & (pos < 16 + cnt[:, None])) | ((pos >= voff) & (pos < voff + 4 * cnt[:, None]))


def bn_backward(grad_out, x, weight, mean, invstd, training):
    """native_batch_norm_backward as the reference calls it on the dequantised input (exact/exact/ops.py:238,
    248-251), in float64: (grad_input, grad_weight, grad_bias).  training: mean / invstd are the batch statistics
    saved by the forward; otherwise the running mean and 1 / sqrt(running_var + eps)."""
    g = np.asarray(grad_out, np.float64)
    xc = np.asarray(x, np.float64) - np.asarray(mean, np.float64)[None, :]
    invstd = np.asarray(invstd, np.float64)
    w = np.ones_like(invstd) if weight is None else np.asarray(weight, np.float64)
    n = g.shape[0]
    sum_g = g.sum(0)
    sum_gx = (g * xc).sum(0)
    if training:
        grad_in = (g - sum_g / n - xc * (invstd * invstd * sum_gx / n)) * (invstd * w)
    else:
        grad_in = g * (invstd * w)
    return grad_in, sum_gx * invstd, sum_g


def _u16(a):
    a = np.asarray(a)
    if a.dtype == np.float16:
        a = a.view(np.uint16)
    return np.ascontiguousarray(a, dtype=np.uint16)


def quantize_activation_f16(x, noise, bits):
    """ops.py:69-83 for an fp16 activation (statistics stay fp16, ops.py:82-83) -> (packed u8, scale f16, min f16),
    with the half arithmetic of the reference's half kernels and of torch's half tensor ops."""
    xb, noise = _u16(x), _f32(noise)
    N, D = xb.shape
    mn, sc = np.empty(N, np.uint16), np.empty(N, np.uint16)
    lib().orc_row_stats_f16(_p(xb), i64(N), i64(D), cint(bits), _p(mn), _p(sc))
    packed = np.empty(packed_nbytes(N, D, bits), np.uint8)
    lib().orc_pack_f16(_p(xb), _p(mn), _p(sc), _p(noise), i64(N), i64(D), cint(bits), _p(packed))
    return packed, sc.view(np.float16), mn.view(np.float16)


def pack_f16(x, mn, scale, noise, bits):
    """pack_single_precision on halves (quantization_cuda_kernel.cu:73-93, scalar_t = Half)."""
    xb, noise = _u16(x), _f32(noise)
    N, D = xb.shape
    packed = np.empty(packed_nbytes(N, D, bits), np.uint8)
    lib().orc_pack_f16(_p(xb), _p(_u16(mn)), _p(_u16(scale)), _p(noise), i64(N), i64(D), cint(bits), _p(packed))
    return packed


def unpack_f16(packed, scale, mn, N, D, bits):
    """unpack_single_precision with half statistics (quantization_cuda_kernel.cu:167-184) -> fp16 [N, D]."""
    packed = np.ascontiguousarray(packed).view(np.uint8)
    out = np.empty((N, D), np.uint16)
    lib().orc_unpack_f16(_p(packed), _p(_u16(scale)), _p(_u16(mn)), i64(N), i64(D), cint(bits), _p(out))
    return out.view(np.float16)


def spmm_f16(rowptr, col, val, mat, reduce="sum"):
    """CSR x dense on halves with the half arithmetic of the reference's half instantiation (spmm_cuda.cu:142,
    83-92; reducer.cuh:53-77): every product, every partial sum and the mean's divisor rounded to half."""
    rowptr = np.ascontiguousarray(rowptr, dtype=np.int64)
    col = np.ascontiguousarray(col, dtype=np.int64)
    val = None if val is None else _u16(val)
    mat = _u16(mat)
    M, K = rowptr.size - 1, mat.shape[1]
    out = np.empty((M, K), np.uint16)
    lib().orc_spmm_f16(_p(rowptr), _p(col), _p(val), _p(mat), i64(M), i64(K), cint({"sum": 0, "mean": 1}[reduce]), _p(out))
    return out.view(np.float16)


def rows_scale_colsum(g, rowscale=None, pad_to=4):
    """(g * rowscale[:, None] in fp32, zero-padded to a multiple of `pad_to` columns; g.sum(0) in float64): the
    operand D^-1 g of the transposed mean aggregation (spmm.cc:128-137: the weights 1 / max(count, 1) applied to the
    rows of the gradient) and the bias gradient grad_output.sum(0) (backward_func.cc:88-90)."""
    g = _f32(g)
    N, K = g.shape
    Kout = (K + pad_to - 1) // pad_to * pad_to
    out = np.zeros((N, Kout), np.float32)
    out[:, :K] = g if rowscale is None else g * _f32(rowscale)[:, None]
    return out, g.astype(np.float64).sum(0)
