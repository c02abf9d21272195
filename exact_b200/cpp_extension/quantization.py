"""Stand-in for the reference's `exact.cpp_extension.quantization` module
(exact/exact/cpp_extension/quantization.cc:137-143): same function names and argument meaning, each
call forwarded to libexact_b200.so through the C ABI."""
import torch

from .. import _lib
from ..conf import config


def _check_cuda_float(t, name, dim=None, dtypes=(torch.float32,)):
    # ext_common.h:2-32: CUDA, contiguous, rank, dtype
    if not t.is_cuda:
        raise RuntimeError(f"{name} must be a CUDA tensor!")
    if not t.is_contiguous():
        raise RuntimeError(f"{name} must be contiguous!")
    if dim is not None and t.dim() != dim:
        raise RuntimeError(f"The dimension of {name} is not correct!")
    if t.dtype not in dtypes:
        raise RuntimeError(f"The type of {name} is not correct!")


def _dt(t):
    return _lib.DTYPE_F32 if t.dtype == torch.float32 else _lib.DTYPE_BF16


def packed_numel(N, D, bits):
    """Elements of the int8 tensor the reference returns: ceil(N/(8/bits))*D + 1
    (quantization_cuda_kernel.cu:110-113)."""
    return int(_lib.load().exact_packed_bytes(N, D, bits)) + 1


def quantize_pack(data, bits, noise=None, seed=None, offset=None, row_offset=None, want_f32_stats=False):
    """Fused row statistics + stochastic quantise + bit-pack.  One kernel, one read of `data`.
    -> (packed int8 [G*D+1], scale bf16 [N], min bf16 [N][, scale f32, min f32])."""
    _check_cuda_float(data, "data", 2, (torch.float32, torch.bfloat16, torch.float16))
    if bits not in (1, 2, 4, 8):
        raise RuntimeError("bits must be 1, 2, 4 or 8")
    N, D = data.shape
    if noise is not None:
        _check_cuda_float(noise, "noise", 2)
        if tuple(noise.shape) != (N, D):
            raise RuntimeError("noise must have the shape of data")
    lib = _lib.load()
    packed = torch.empty(packed_numel(N, D, bits), dtype=torch.int8, device=data.device)
    if data.dtype == torch.float16:
        # half arithmetic of the reference's half kernels; the statistics stay fp16 (ops.py:82-83)
        if want_f32_stats:
            raise RuntimeError("fp16 activations have fp16 statistics only")
        scale = torch.empty(N, dtype=torch.float16, device=data.device)
        mn = torch.empty(N, dtype=torch.float16, device=data.device)
        if noise is None:
            seed = config.seed if seed is None else seed
            offset = config.next_offset() if offset is None else offset
        else:
            seed = offset = 0
        row_offset = config.row_offset if row_offset is None else row_offset
        _lib.invoke("exact_quantize_pack_f16", 2 * N * D * 2 + packed.numel() - 1 + 4 * N, _lib.ptr(data), N, D, bits,
                    _lib.ptr(noise), seed, offset, row_offset, _lib.ptr(packed), _lib.ptr(scale), _lib.ptr(mn),
                    _lib.stream_ptr())
        return packed, scale, mn
    scale = torch.empty(N, dtype=torch.bfloat16, device=data.device)
    mn = torch.empty(N, dtype=torch.bfloat16, device=data.device)
    sf = mf = None
    if want_f32_stats:
        sf = torch.empty(N, dtype=torch.float32, device=data.device)
        mf = torch.empty(N, dtype=torch.float32, device=data.device)
    if noise is None:
        seed = config.seed if seed is None else seed
        offset = config.next_offset() if offset is None else offset
    else:
        seed = offset = 0
    row_offset = config.row_offset if row_offset is None else row_offset
    nbytes = N * D * data.element_size() + packed.numel() - 1 + 4 * N
    _lib.invoke("exact_quantize_pack", nbytes, _lib.ptr(data), _dt(data), N, D, bits, _lib.ptr(noise), seed,
                offset, row_offset, _lib.ptr(packed), _lib.ptr(scale), _lib.ptr(mn), _lib.ptr(sf), _lib.ptr(mf),
                _lib.stream_ptr())
    if want_f32_stats:
        return packed, scale, mn, sf, mf
    return packed, scale, mn


def rp_supported(D, k, dtype=torch.float32):
    """Shapes the fused projection+pack kernel takes (others use the unfused chain): fp32 rows of any
    length (rows that are not 16-byte aligned are copied in by cp.async instead of TMA), k up to 512 as long
    as three pipeline stages of a [128 x 32] A tile and a [k x 32] sign tile fit in shared memory."""
    kpad = (k + 15) // 16 * 16
    stage = 128 * 128 + kpad * 128
    return dtype == torch.float32 and kpad <= 512 and 200 * 1024 // stage >= (3 if D % 4 else 2)


def rp_quantize_pack(data, R, bits, seed=None, offset=None, row_offset=None, want_projection=False):
    """Fused (data @ R) -> row statistics -> stochastic quantise -> pack, one tcgen05 kernel.
    data [N, D] fp32, R [D, k] = +-1/sqrt(k).  -> (packed int8 [G*k+1], scale bf16 [N], min bf16 [N][, y fp32 [N,k]])."""
    _check_cuda_float(data, "data", 2)
    _check_cuda_float(R, "R", 2)
    N, D = data.shape
    k = R.shape[1]
    if R.shape[0] != D:
        raise RuntimeError("R must be [D, k]")
    if bits not in (1, 2, 4, 8):
        raise RuntimeError("bits must be 1, 2, 4 or 8")
    if not rp_supported(D, k) or data.data_ptr() % 4 != 0:
        raise _lib.ExactB200Error("rp_quantize_pack: unsupported shape (needs fp32 and k <= 512)")
    lib = _lib.load()
    ws = torch.empty(int(lib.exact_rp_workspace_bytes(D, k)), dtype=torch.uint8, device=data.device)
    packed = torch.empty(packed_numel(N, k, bits), dtype=torch.int8, device=data.device)
    scale = torch.empty(N, dtype=torch.bfloat16, device=data.device)
    mn = torch.empty(N, dtype=torch.bfloat16, device=data.device)
    y = torch.empty((N, k), dtype=torch.float32, device=data.device) if want_projection else None
    seed = config.seed if seed is None else seed
    offset = config.next_offset() if offset is None else offset
    row_offset = config.row_offset if row_offset is None else row_offset
    nbytes = N * D * 4 + D * k * 4 + packed.numel() - 1 + 4 * N
    _lib.invoke("exact_rp_quantize_pack", nbytes, _lib.ptr(data), N, D, _lib.ptr(R), k, bits, seed, offset,
                row_offset, _lib.ptr(ws), _lib.ptr(packed), _lib.ptr(scale), _lib.ptr(mn), _lib.ptr(y),
                _lib.stream_ptr())
    if config.check_device_status:
        status = int(ws[:4].view(torch.int32).item())
        if status != 0:
            raise _lib.ExactB200Error(f"rp_quantize_pack: device status {status} (a bounded on-chip wait expired)")
    return (packed, scale, mn, y) if want_projection else (packed, scale, mn)


def unpack_rp_supported(D, k):
    """Shapes the fused unpack+transpose-projection kernels take: every configured one (sign(R) resident when it
    fits beside the A tiles, streamed in panels otherwise)."""
    Dpad, kpad = (D + 15) // 16 * 16, (k + 31) // 32 * 32
    return D > 0 and k > 0 and Dpad * kpad < (1 << 28)


def unpack_dequant_rp(packed, bits, scale, mn, N, R):
    """Fused dequantise(packed [N, k]) @ R^T -> fp32 [N, D]; R is [D, k] = +-1/sqrt(k)."""
    if not packed.is_cuda or packed.dtype != torch.int8 or packed.dim() != 1:
        raise RuntimeError("The type of data is not correct!")
    _check_cuda_float(scale, "scale", 1, (torch.bfloat16,))
    _check_cuda_float(mn, "min", 1, (torch.bfloat16,))
    _check_cuda_float(R, "R", 2)
    D, k = R.shape
    if not unpack_rp_supported(D, k):
        raise _lib.ExactB200Error("unpack_dequant_rp: unsupported shape")
    lib = _lib.load()
    need = int(lib.exact_packed_bytes(N, k, bits))
    if packed.numel() < need or scale.numel() < N or mn.numel() < N:
        raise RuntimeError("packed stream or statistics shorter than N x k requires")
    ws = torch.empty(int(lib.exact_unpack_rp_workspace_bytes(D, k)), dtype=torch.uint8, device=packed.device)
    out = torch.empty((N, D), dtype=torch.float32, device=packed.device)
    nbytes = need + 4 * N + D * k * 4 + N * D * 4
    _lib.invoke("exact_unpack_dequant_rp", nbytes, _lib.ptr(packed), bits, _lib.ptr(scale), _lib.ptr(mn), N, k,
                _lib.ptr(R), D, _lib.ptr(ws), _lib.ptr(out), _lib.stream_ptr())
    if config.check_device_status:
        status = int(ws[:4].view(torch.int32).item())
        if status != 0:
            raise _lib.ExactB200Error(f"unpack_dequant_rp: device status {status} (a bounded on-chip wait expired)")
    return out


def pack_single_precision(data, min, max, scale, bits, stochastic, noise=None, seed=None, offset=None,
                          row_offset=None):
    """quantization.cc:37-48.  `max` is accepted and ignored, as in the reference kernel; `stochastic`
    must be true (quantization_cuda_kernel.cu:123).  `noise` (optional, [N,D] fp32) replaces the
    Philox draw."""
    _check_cuda_float(data, "data", 2, (torch.float32, torch.bfloat16, torch.float16))
    half = data.dtype == torch.float16   # the reference's half instantiation: statistics are halves too
    stat_types = (torch.float16,) if half else (torch.float32,)
    _check_cuda_float(min, "min", 1, stat_types)
    _check_cuda_float(max, "max", 1, stat_types)
    _check_cuda_float(scale, "scale", 1, stat_types)
    if 8 % bits != 0 or bits not in (1, 2, 4, 8):
        raise RuntimeError("bits must be 1, 2, 4 or 8")
    if not stochastic:
        raise RuntimeError("stochastic must be true")
    N, D = data.shape
    packed = torch.empty(packed_numel(N, D, bits), dtype=torch.int8, device=data.device)
    if noise is None:
        seed = config.seed if seed is None else seed
        offset = config.next_offset() if offset is None else offset
    else:
        seed = offset = 0
    row_offset = config.row_offset if row_offset is None else row_offset
    if half:
        _lib.invoke("exact_pack_single_precision_f16", N * D * 2 + packed.numel() - 1 + 4 * N, _lib.ptr(data),
                    _lib.ptr(min), _lib.ptr(scale), N, D, bits, _lib.ptr(noise), seed, offset, row_offset,
                    _lib.ptr(packed), _lib.stream_ptr())
        return packed
    nbytes = N * D * data.element_size() + packed.numel() - 1 + 8 * N
    _lib.invoke("exact_pack_single_precision", nbytes, _lib.ptr(data), _dt(data), _lib.ptr(min), _lib.ptr(scale),
                N, D, bits, _lib.ptr(noise), seed, offset, row_offset, _lib.ptr(packed), _lib.stream_ptr())
    return packed


def unpack_single_precision(data, bits, scale, min, N, group_size):
    """quantization.cc:50-62.  scale/min may be fp32 (reference signature), bf16 (the stored statistics of an
    fp32 activation; widening happens in the kernel) or fp16 (an fp16 activation).  Returns [N, group_size] in
    fp32, or in fp16 for fp16 statistics."""
    if not data.is_cuda or not data.is_contiguous() or data.dim() != 1 or data.dtype != torch.int8:
        raise RuntimeError("The type of data is not correct!")
    _check_cuda_float(scale, "scale", 1, (torch.float32, torch.bfloat16, torch.float16))
    _check_cuda_float(min, "min", 1, (torch.float32, torch.bfloat16, torch.float16))
    if scale.dtype != min.dtype:
        raise RuntimeError("scale and min must have the same dtype")
    if bits not in (1, 2, 4, 8):
        raise RuntimeError("bits must be 1, 2, 4 or 8")
    lib = _lib.load()
    need = int(lib.exact_packed_bytes(N, group_size, bits))
    if data.numel() < need or scale.numel() < N or min.numel() < N:
        raise RuntimeError("packed stream or statistics shorter than N x group_size requires")
    if scale.dtype == torch.float16:
        # the output has the statistics' dtype (quantization_cuda_kernel.cu:194-195): fp16, half arithmetic
        out = torch.empty((N, group_size), dtype=torch.float16, device=data.device)
        _lib.invoke("exact_unpack_single_precision_f16", need + 4 * N + 2 * N * group_size, _lib.ptr(data), bits,
                    _lib.ptr(scale), _lib.ptr(min), N, group_size, _lib.ptr(out), _lib.stream_ptr())
        return out
    out = torch.empty((N, group_size), dtype=torch.float32, device=data.device)
    nbytes = need + 2 * N * scale.element_size() + 4 * N * group_size
    _lib.invoke("exact_unpack_single_precision", nbytes, _lib.ptr(data), bits, _lib.ptr(scale), _lib.ptr(min),
                _dt(scale), N, group_size, _lib.ptr(out), _lib.stream_ptr())
    return out


ACT_RELU, ACT_DROPOUT, ACT_RELU_DROPOUT, ACT_LEAKY_RELU = 0, 1, 2, 3   # EXACT_ACT_*
_ACT_DTYPES = (torch.float32, torch.float16)


def _act_forward_f16(op, input, param, uniforms, seed, offset, index_offset, out, mask):
    """fp16 tensors: the reference's half instantiations (fp32 arithmetic on widened values, one rounding on
    the store)."""
    n = input.numel()
    _lib.invoke("exact_act_quantized_forward_f16", 4 * n + n // 8, op, _lib.ptr(input), n, param, _lib.ptr(uniforms),
                seed, offset, index_offset, _lib.ptr(out), _lib.ptr(mask), _lib.stream_ptr())


def _act_backward_f16(op, grad_output, mask, param, gin):
    n = grad_output.numel()
    _lib.invoke("exact_act_quantized_backward_f16", 4 * n + n // 8, op, _lib.ptr(grad_output), _lib.ptr(mask), n, param,
                _lib.ptr(gin), _lib.stream_ptr())


class _ActQuantizedReLU(torch.autograd.Function):
    """quantization.cc:66-79."""

    @staticmethod
    def forward(ctx, input):
        lib = _lib.load()
        n = input.numel()
        out = torch.empty_like(input)
        mask = torch.empty(int(lib.exact_mask_words(n)), dtype=torch.int32, device=input.device)
        if input.dtype == torch.float16:
            _act_forward_f16(ACT_RELU, input, 0.0, None, 0, 0, 0, out, mask)
        else:
            _lib.invoke("exact_act_quantized_relu_forward", 8 * n + n // 8, _lib.ptr(input), n, _lib.ptr(out),
                        _lib.ptr(mask), _lib.stream_ptr())
        ctx.save_for_backward(mask)
        return out

    @staticmethod
    def backward(ctx, grad_output):
        (mask,) = ctx.saved_tensors
        grad_output = grad_output.contiguous()
        gin = torch.empty_like(grad_output)
        n = grad_output.numel()
        if grad_output.dtype == torch.float16:
            _act_backward_f16(ACT_RELU, grad_output, mask, 0.0, gin)
        else:
            _lib.invoke("exact_act_quantized_relu_backward", 8 * n + n // 8, _lib.ptr(grad_output), _lib.ptr(mask), n,
                        _lib.ptr(gin), _lib.stream_ptr())
        return gin


def act_quantized_relu(input):
    """quantization.cc:81-84."""
    _check_cuda_float(input, "input", None, _ACT_DTYPES)
    return _ActQuantizedReLU.apply(input)


class _ActQuantizedDropout(torch.autograd.Function):
    """quantization.cc:111-129."""

    @staticmethod
    def forward(ctx, input, p, uniforms):
        lib = _lib.load()
        n = input.numel()
        out = torch.empty_like(input)
        mask = torch.empty(int(lib.exact_mask_words(n)), dtype=torch.int32, device=input.device)
        if uniforms is None:
            seed, offset = config.seed, config.next_offset()
        else:
            seed = offset = 0
        # rows are the sharded dimension: element 0 of this shard is global element row_offset * row_len
        index_offset = config.row_offset * (n // input.shape[0]) if (input.dim() >= 2 and n) else 0
        if input.dtype == torch.float16:
            _act_forward_f16(ACT_DROPOUT, input, p, uniforms, seed, offset, index_offset, out, mask)
        else:
            _lib.invoke("exact_act_quantized_dropout_forward", 8 * n + n // 8, _lib.ptr(input), n, p,
                        _lib.ptr(uniforms), seed, offset, index_offset, _lib.ptr(out), _lib.ptr(mask),
                        _lib.stream_ptr())
        ctx.save_for_backward(mask)
        ctx.p = p
        return out

    @staticmethod
    def backward(ctx, grad_output):
        (mask,) = ctx.saved_tensors
        grad_output = grad_output.contiguous()
        gin = torch.empty_like(grad_output)
        n = grad_output.numel()
        if grad_output.dtype == torch.float16:
            _act_backward_f16(ACT_DROPOUT, grad_output, mask, ctx.p, gin)
        else:
            _lib.invoke("exact_act_quantized_dropout_backward", 8 * n + n // 8, _lib.ptr(grad_output), _lib.ptr(mask),
                        n, ctx.p, _lib.ptr(gin), _lib.stream_ptr())
        return gin, None, None


def act_quantized_dropout(input, p, train, uniforms=None):
    """quantization.cc:131-134; eval mode returns the input tensor itself (quantization.cc:115-117).
    `uniforms` (optional, fp32, shape of input) replaces the Philox draw."""
    _check_cuda_float(input, "input", None, _ACT_DTYPES)
    if not train:
        return input
    if uniforms is not None:
        _check_cuda_float(uniforms, "uniforms")
        if uniforms.numel() != input.numel():
            raise RuntimeError("uniforms must have the shape of input")
    return _ActQuantizedDropout.apply(input, float(p), uniforms)


class _ActQuantizedReLUDropout(_ActQuantizedDropout):
    """ReLU then dropout in one pass, one mask; the backward is the dropout's with that mask."""

    @staticmethod
    def forward(ctx, input, p, uniforms):
        lib = _lib.load()
        n = input.numel()
        out = torch.empty_like(input)
        mask = torch.empty(int(lib.exact_mask_words(n)), dtype=torch.int32, device=input.device)
        if uniforms is None:
            seed, offset = config.seed, config.next_offset()
        else:
            seed = offset = 0
        index_offset = config.row_offset * (n // input.shape[0]) if (input.dim() >= 2 and n) else 0
        if input.dtype == torch.float16:
            _act_forward_f16(ACT_RELU_DROPOUT, input, p, uniforms, seed, offset, index_offset, out, mask)
        else:
            _lib.invoke("exact_act_quantized_relu_dropout_forward", 8 * n + n // 8, _lib.ptr(input), n, p,
                        _lib.ptr(uniforms), seed, offset, index_offset, _lib.ptr(out), _lib.ptr(mask),
                        _lib.stream_ptr())
        ctx.save_for_backward(mask)
        ctx.p = p
        return out


def act_quantized_relu_dropout(input, p, train, uniforms=None):
    """dropout(relu(input)) as the two reference ops compute it (quantization.cc:66-84, 111-134), in one
    pass and with one saved mask.  Eval mode: relu only."""
    _check_cuda_float(input, "input", None, _ACT_DTYPES)
    if not train:
        return torch.relu(input)
    if uniforms is not None:
        _check_cuda_float(uniforms, "uniforms")
        if uniforms.numel() != input.numel():
            raise RuntimeError("uniforms must have the shape of input")
    return _ActQuantizedReLUDropout.apply(input.contiguous(), float(p), uniforms)


class _ActQuantizedLeakyReLU(torch.autograd.Function):
    """quantization.cc:87-107."""

    @staticmethod
    def forward(ctx, input, slope):
        lib = _lib.load()
        n = input.numel()
        out = torch.empty_like(input)
        mask = torch.empty(int(lib.exact_mask_words(n)), dtype=torch.int32, device=input.device)
        if input.dtype == torch.float16:
            _act_forward_f16(ACT_LEAKY_RELU, input, slope, None, 0, 0, 0, out, mask)
        else:
            _lib.invoke("exact_act_quantized_leaky_relu_forward", 8 * n + n // 8, _lib.ptr(input), n, slope,
                        _lib.ptr(out), _lib.ptr(mask), _lib.stream_ptr())
        ctx.save_for_backward(mask)
        ctx.slope = slope
        return out

    @staticmethod
    def backward(ctx, grad_output):
        (mask,) = ctx.saved_tensors
        grad_output = grad_output.contiguous()
        gin = torch.empty_like(grad_output)
        n = grad_output.numel()
        if grad_output.dtype == torch.float16:
            _act_backward_f16(ACT_LEAKY_RELU, grad_output, mask, ctx.slope, gin)
        else:
            _lib.invoke("exact_act_quantized_leaky_relu_backward", 8 * n + n // 8, _lib.ptr(grad_output),
                        _lib.ptr(mask), n, ctx.slope, _lib.ptr(gin), _lib.stream_ptr())
        return gin, None


def act_quantized_leaky_relu(input, slope):
    """quantization.cc:104-107."""
    _check_cuda_float(input, "input", None, _ACT_DTYPES)
    return _ActQuantizedLeakyReLU.apply(input.contiguous(), float(slope))
