"""Stand-in for the reference's `exact.cpp_extension.backward_func` module
(exact/exact/cpp_extension/backward_func.cc:83-107): the dense-layer GEMMs and ATen batch-norm
pass-throughs.  The tall GEMMs (rows = nodes) go to the tensor-core kernel with fp32-equivalent accuracy
(exact_linear_forward); the weight-gradient reductions and unsupported shapes stay library GEMMs."""
import torch

from .. import _lib
from ..conf import config


def _tc_ok(a):
    return (config.linear_tensor_core and a.is_cuda and a.dtype == torch.float32 and a.dim() == 2
            and a.size(0) >= 1024)


def _rows16(a):
    """`a` with 16-byte aligned rows: itself when its pitch already is, else a zero-padded copy."""
    if a.stride(1) == 1 and a.stride(0) % 4 == 0 and a.stride(0) >= a.size(1) and a.data_ptr() % 16 == 0:
        return a
    K = a.size(1)
    out = a.new_zeros((a.size(0), (K + 3) // 4 * 4))
    out[:, :K].copy_(a)
    return out[:, :K]


def linear_forward(a, weight, bias=None, a2=None, weight2=None, out=None, accumulate=False):
    """a @ weight.T (+ a2 @ weight2.T) (+ bias), optionally added to `out`: F.linear of ops.py:150 and the
    g W product of backward_func.cc:86 (pass weight.t()).  fp32 in and out."""
    if not _tc_ok(a) or (a2 is not None and not _tc_ok(a2)):
        _lib.note_library_call("F.linear (rows < 1024, not fp32 or not CUDA)")
        r = torch.nn.functional.linear(a, weight, bias)
        if a2 is not None:
            r = r.addmm_(a2, weight2.t())
        if out is not None:
            return out.add_(r) if accumulate else out.copy_(r)
        return r
    lib = _lib.load()
    M, K = a.shape
    N = weight.size(0)
    a = _rows16(a)
    w = weight if weight.stride(1) == 1 else weight.contiguous()
    K2 = 0
    if a2 is not None:
        K2 = a2.size(1)
        a2 = _rows16(a2)
        w2 = weight2 if weight2.stride(1) == 1 else weight2.contiguous()
    if bias is not None:
        bias = bias.contiguous()
    if out is None:
        out = torch.empty((M, N), dtype=torch.float32, device=a.device)
        accumulate = False
    assert out.shape == (M, N) and out.stride(1) == 1
    for n0 in range(0, N, 256):
        n1 = min(N, n0 + 256)
        ws = torch.empty(int(lib.exact_linear_workspace_bytes(n1 - n0, K, K2)), dtype=torch.uint8, device=a.device)
        wb, cb = w[n0:n1], out[:, n0:n1]
        nbytes = 4 * (M * (K + K2) + (n1 - n0) * (K + K2) + M * (n1 - n0) * (2 if accumulate else 1))
        _lib.invoke("exact_linear_forward", nbytes, _lib.ptr(a), M, K, a.stride(0), _lib.ptr(wb), wb.stride(0),
                    _lib.ptr(a2) if K2 else None, K2, a2.stride(0) if K2 else 0,
                    _lib.ptr(w2[n0:n1]) if K2 else None, w2.stride(0) if K2 else 0, n1 - n0,
                    _lib.ptr(bias[n0:n1]) if bias is not None else None, 1 if accumulate else 0, _lib.ptr(ws),
                    _lib.ptr(cb), out.stride(0), _lib.stream_ptr(), flops=6.0 * M * (K + K2) * (n1 - n0))
        if config.check_device_status:
            status = int(ws[:4].view(torch.int32).item())
            if status != 0:
                raise _lib.ExactB200Error(f"linear_forward: device status {status} (a bounded on-chip wait expired)")
    return out


def rows_reduce_mm(g, x, batches=512):
    """g^T x for g [M, out], x [M, k] with M in the millions and out, k small: the reduction over rows is
    cut into `batches` independent products that one batched library GEMM computes in parallel and a sum
    joins (a single GEMM call leaves most SMs idle on this shape: 2.0 ms against 0.76 ms at
    2.45M x 256 x 32).  Same fp32 arithmetic, pairwise-style summation."""
    M = g.size(0)
    _lib.note_library_call("g^T x on the unpacked activation (library GEMM)")
    if not (g.is_cuda and g.dim() == 2 and M >= 64 * batches and g.is_contiguous() and x.is_contiguous()):
        return g.t().mm(x)
    rows = M // batches * batches
    out = torch.bmm(g[:rows].view(batches, -1, g.size(1)).transpose(1, 2), x[:rows].view(batches, -1, x.size(1))).sum(0)
    if rows < M:
        out.addmm_(g[rows:].t(), x[rows:])
    return out


def grad_weight_supported(g, k0, k1, bits):
    """Shapes exact_grad_weight_from_packed takes: fp32 g [N, O] with O <= 256 (padded to a multiple of 4), at least 4,096 rows
    (below that the library GEMM on the unpacked activation is as fast), and few enough activation columns for
    four producer warps (k0 + k1 <= 1024 * bits / 256)."""
    if not (config.grad_weight_tensor_core and g.is_cuda and g.dtype == torch.float32 and g.dim() == 2):
        return False
    N, O = g.shape
    kpad = (k0 + 15) // 16 * 16 + ((k1 + 15) // 16 * 16 if k1 else 0)
    # a width that is not a multiple of 4 (47 classes) goes in as a zero-padded copy of g
    return (N >= 4096 and (O + 3) // 4 * 4 <= 256 and kpad <= 256 and (k0 + k1) * (32 // (8 // bits)) <= 1024
            and g.is_contiguous() and (g.data_ptr() % 16 == 0 or O % 4 != 0))


_SM_COUNT = {}


def grad_weight_from_packed(g, q0, k0, q1=None, k1=0):
    """(g^T Xq0 [O, k0], g^T Xq1 [O, k1] or None) for packed activations q = (packed, bits, scale_bf16, min_bf16)
    of N rows: backward_func.cc:87 with the dequantisation of ops.py:164 folded in, one pass over g."""
    lib = _lib.load()
    N, O_true = g.shape
    if O_true % 4:
        gp = g.new_zeros((N, (O_true + 3) // 4 * 4))
        gp[:, :O_true].copy_(g)
        g = gp
    N, O = g.shape
    bits = q0[1]
    k0pad = (k0 + 15) // 16 * 16
    kpad = k0pad + ((k1 + 15) // 16 * 16 if q1 is not None else 0)
    dev = g.device
    sms = _SM_COUNT.get(dev.index)
    if sms is None:
        sms = _SM_COUNT[dev.index] = torch.cuda.get_device_properties(dev).multi_processor_count
    ws_bytes = int(lib.exact_grad_weight_workspace_bytes(O, kpad, sms))
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device=dev)
    out = torch.empty((O, kpad), dtype=torch.float32, device=dev)
    nbytes = 4 * N * O + (N * (k0 + (k1 if q1 is not None else 0)) * bits) // 8 + 4 * N * (2 if q1 is not None else 1)
    _lib.invoke("exact_grad_weight_from_packed", nbytes, _lib.ptr(g), N, O, _lib.ptr(q0[0]), _lib.ptr(q0[2]), _lib.ptr(q0[3]),
                k0, _lib.ptr(q1[0]) if q1 is not None else None, _lib.ptr(q1[2]) if q1 is not None else None,
                _lib.ptr(q1[3]) if q1 is not None else None, k1 if q1 is not None else 0, bits, _lib.ptr(ws), ws_bytes,
                _lib.ptr(out), kpad, _lib.stream_ptr(), flops=2.0 * N * O * kpad)
    if config.check_device_status:
        status = int(ws[:4].view(torch.int32).item())
        if status != 0:
            raise _lib.ExactB200Error(f"grad_weight_from_packed: device status {status} (a bounded on-chip wait expired)")
    return out[:O_true, :k0], (out[:O_true, k0pad:k0pad + k1] if q1 is not None else None)


def linear_backward(grad_output, input, weight, bias=None, need_grad_input=True):
    """backward_func.cc:83-93.  The input gradient is left out (None) when the caller has no use for it."""
    grad_input = linear_forward(grad_output, weight.t()) if need_grad_input else None
    grad_weight = rows_reduce_mm(grad_output, input)
    grad_bias = rows_scale_colsum(grad_output)[1] if bias is not None else None
    return grad_input, grad_weight, grad_bias


def native_batch_norm(input, weight, bias, running_mean, running_var, training, momentum, eps):
    return torch.ops.aten.native_batch_norm(input, weight, bias, running_mean, running_var, training, momentum, eps)


def _batch_norm_impl_index(input, weight, bias, running_mean, running_var, training, momentum, eps, cudnn_enabled):
    return torch.ops.aten._batch_norm_impl_index(input, weight, bias, running_mean, running_var, training,
                                                 momentum, eps, cudnn_enabled)


def native_batch_norm_backward(grad_out, input, weight, running_mean, running_var, save_mean, save_invstd,
                               train, eps, output_mask):
    return torch.ops.aten.native_batch_norm_backward(grad_out, input, weight, running_mean, running_var,
                                                     save_mean, save_invstd, train, eps, output_mask)


def batch_norm_backward_from_packed_supported(grad_out, quantized):
    """Whether native_batch_norm_backward can read the saved input in its packed form (this library's kernels):
    a compressed [N, D] fp32 activation with bf16 row statistics and D a multiple of 4."""
    q_input, q_bits, q_scale, q_min = quantized
    return (q_bits is not None and grad_out.is_cuda and grad_out.dtype == torch.float32 and grad_out.dim() == 2
            and grad_out.size(1) % 4 == 0 and q_scale.dtype == torch.bfloat16 and q_input.is_cuda)


def batch_norm_backward_from_packed(grad_out, quantized, weight, running_mean, running_var, save_mean, save_invstd,
                                    train, eps, output_mask):
    """native_batch_norm_backward (the call of ops.py:248-251) with the dequantisation of ops.py:238 folded into
    both of its passes: the column sums and the element-wise pass read the packed bytes and the bf16 row
    statistics, the [N, D] reconstruction is never written.  Returns (grad_input, grad_weight, grad_bias)."""
    q_input, q_bits, q_scale, q_min = quantized
    g = grad_out.contiguous()
    N, D = g.shape
    if train:
        mean, invstd = save_mean, save_invstd
    else:
        mean, invstd = running_mean, torch.rsqrt(running_var + eps)
    mean, invstd = mean.to(torch.float32).contiguous(), invstd.to(torch.float32).contiguous()
    w = None if weight is None else weight.detach().to(torch.float32).contiguous()
    lib = _lib.load()
    ws_bytes = int(lib.exact_bn_backward_workspace_bytes(D))
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device=g.device)
    grad_input = torch.empty_like(g) if output_mask[0] else None
    grad_weight = torch.empty(D, dtype=torch.float32, device=g.device) if output_mask[1] else None
    grad_bias = torch.empty(D, dtype=torch.float32, device=g.device) if output_mask[2] else None
    wpt = 8 // q_bits
    nbytes = (2 if (grad_input is not None and (train or grad_weight is not None or grad_bias is not None)) else 1) * (
        N * D * 4 + (N + wpt - 1) // wpt * D + 4 * N) + (N * D * 4 if grad_input is not None else 0)
    _lib.invoke("exact_bn_backward_from_packed", nbytes, _lib.ptr(g), N, D, _lib.ptr(q_input), q_bits, _lib.ptr(q_scale),
                _lib.ptr(q_min), _lib.ptr(w), _lib.ptr(mean), _lib.ptr(invstd), 1 if train else 0, _lib.ptr(ws), ws_bytes,
                _lib.ptr(grad_input), _lib.ptr(grad_weight), _lib.ptr(grad_bias), _lib.stream_ptr())
    return grad_input, grad_weight, grad_bias


def rows_scale_colsum(g, rowscale=None, want_scaled=False, want_colsum=True, pad_to=4):
    """One pass over g [N, K] -> (g * rowscale[:, None] zero-padded to a multiple of `pad_to` columns or None,
    g.sum(0) or None): the operand D^-1 g of the transposed mean aggregation (spmm.cc:128-137) and the bias gradient
    (backward_func.cc:88-90).  Small or non-fp32 inputs take the framework's ops."""
    N, K = g.shape
    if not (g.is_cuda and g.dtype == torch.float32 and g.dim() == 2 and g.stride(1) == 1 and N >= 1024):
        scaled = None
        if want_scaled:
            scaled = g.new_zeros((N, (K + pad_to - 1) // pad_to * pad_to))
            scaled[:, :K] = g if rowscale is None else g * rowscale.unsqueeze(1)
        return scaled, (g.sum(0) if want_colsum else None)
    lib = _lib.load()
    Kout = (K + pad_to - 1) // pad_to * pad_to if want_scaled else K
    out = torch.empty((N, Kout), dtype=torch.float32, device=g.device) if want_scaled else None
    colsum = torch.empty(K, dtype=torch.float32, device=g.device) if want_colsum else None
    ws_bytes = int(lib.exact_rows_scale_colsum_workspace_bytes(Kout)) if want_colsum else 0
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device=g.device) if want_colsum else None
    if rowscale is not None:
        rowscale = rowscale.to(torch.float32).contiguous()
    nbytes = 4 * N * K + (4 * N * Kout if want_scaled else 0)
    _lib.invoke("exact_rows_scale_colsum", nbytes, _lib.ptr(g), N, K, g.stride(0), _lib.ptr(rowscale), _lib.ptr(out), Kout,
                Kout, _lib.ptr(colsum), _lib.ptr(ws), ws_bytes, _lib.stream_ptr())
    return out, colsum
