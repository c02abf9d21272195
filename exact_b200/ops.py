"""Autograd Functions and helpers of the compressed-activation path, with the names, arguments and
return values of the reference's exact/exact/ops.py.  Arithmetic runs in libexact_b200.so; dense
GEMMs and batch norm stay library calls, as in the reference."""
import numpy as np
import torch
from torch.amp import custom_bwd, custom_fwd
import torch.nn.functional as F
from torch.autograd.function import Function

from . import _lib
from .conf import config
from .cpp_extension import backward_func as ext_backward_func
from .cpp_extension import quantization as ext_quantization
from .cpp_extension import spmm
from .utils import empty_cache, swap_to_cpu


def quantize_and_pack(data, bits, mn, mx, noise=None):
    """ops.py:20-43: (data [N,D], bits, row min, row max) -> (packed, scale)."""
    if config.simulate:
        # ops.py:21-34: unpacked integer codes with a widened range; a debugging mode in torch ops.
        B = 2 ** bits - 1
        mn = mn - 1e-6
        mx = mx + 1e-6
        scale = B / (mx - mn)
        output = (data - mn.view(-1, 1)) * scale.view(-1, 1)
        if config.stochastic:
            output = output + (output.new_empty(output.shape).uniform_(-0.5, 0.5) if noise is None else noise - 0.5)
        output = F.relu(output).round_().int()
        return output, scale
    assert type(bits) == int
    scale = (2 ** bits - 1) / (mx - mn)
    output = ext_quantization.pack_single_precision(data, mn, mx, scale.to(torch.float32), bits,
                                                    config.stochastic, noise=noise)
    if config.swap:
        output = swap_to_cpu(output)
    return output, scale


def dequantize_and_unpack(data, shape, bits, scale, mn):
    """ops.py:46-58."""
    if config.simulate:
        return data / scale.view(-1, 1) + mn.view(-1, 1)
    if config.swap:
        data = data.cuda()
    N = shape[0]
    num_features = int(np.prod(shape[1:]))
    assert type(bits) == int
    return ext_quantization.unpack_single_precision(data, bits, scale, mn, N, num_features)


def no_scheme_compute_quantization_bits(input):
    """ops.py:61-66."""
    N = input.shape[0]
    input_flatten = input.view(N, -1)
    mn, mx = torch.min(input_flatten, 1)[0], torch.max(input_flatten, 1)[0]
    b = config.activation_compression_bits[0]
    return input_flatten, b, mn, mx


def quantize_activation(input, scheme, noise=None):
    """ops.py:69-83 -> (q_input int8 [ceil(N/(8/b))*D + 1], q_bits, q_scale bf16 [N], q_min bf16 [N]), or
    (input, None, None, None) when compression is off.  An fp16 activation (AMP: ops.py:130) keeps fp16
    statistics (ops.py:82-83) and is quantised with the half arithmetic of the reference's half kernels.

    The row min/max, the scale, the stochastic quantise + pack and the bf16 rounding of the
    statistics run as ONE kernel that reads `input` once.  `noise` ([N, D] fp32 in [0,1)) replaces
    the Philox draw; with it the result is bit-identical to the reference's chain of ops."""
    if not config.compress_activation:
        if config.swap:
            input = swap_to_cpu(input)
        return input, None, None, None
    if config.simulate:
        if scheme:
            input_groups, q_bits, q_min, mx = scheme.compute_quantization_bits(input)
        else:
            input_groups, q_bits, q_min, mx = no_scheme_compute_quantization_bits(input)
        q_input, q_scale = quantize_and_pack(input_groups, q_bits, q_min, mx, noise)
        return q_input, q_bits, q_scale.to(torch.bfloat16), q_min.to(torch.bfloat16)
    if input.dtype not in (torch.float32, torch.bfloat16, torch.float16):
        raise NotImplementedError("quantize_activation: fp32, bf16 and fp16 activations are supported")
    if not config.stochastic:
        raise RuntimeError("stochastic must be true")  # quantization_cuda_kernel.cu:123
    q_bits = config.activation_compression_bits[0]
    N = input.shape[0]
    flat = input.reshape(N, -1)
    if not flat.is_contiguous():
        flat = flat.contiguous()
    if noise is not None:
        noise = noise.reshape(N, -1)
    q_input, q_scale, q_min = ext_quantization.quantize_pack(flat, q_bits, noise=noise)
    if config.swap:
        q_input = swap_to_cpu(q_input)
    return q_input, q_bits, q_scale, q_min


def dequantize_activation(quantized, q_input_shape):
    """ops.py:86-98.  The bf16 statistics are widened inside the unpack kernel."""
    if not config.compress_activation:
        ret = quantized[0]
        if config.swap:
            ret = ret.cuda(non_blocking=True)
        return ret
    q_input, q_bits, q_scale, q_min = quantized
    if config.simulate and q_scale.dtype == torch.bfloat16:
        q_scale = q_scale.to(torch.float32)
        q_min = q_min.to(torch.float32)
    input = dequantize_and_unpack(q_input, q_input_shape, q_bits, q_scale, q_min)
    return input.contiguous()


def _rademacher(rows, cols, device, dtype, seed=None, offset=None):
    """R[D,k] = +-1/sqrt(k) (ops.py:112-114).  The signs come from Philox keyed by (config.seed, offset)
    instead of torch's global CUDA generator, so every rank of a row-sharded run draws the same R."""
    out = torch.empty((rows, cols), dtype=torch.float32, device=device)
    seed = config.seed if seed is None else seed
    offset = config.next_offset() if offset is None else offset
    _lib.invoke("exact_rademacher", rows * cols * 4, seed, offset, rows, cols, _lib.ptr(out), _lib.stream_ptr())
    return out if dtype == torch.float32 else out.to(dtype)


@torch.no_grad()
def input2rp(input, kept_acts):
    """ops.py:107-118 -> (input @ R, R)."""
    assert len(input.size()) == 2
    rand_matrix = _rademacher(input.shape[1], kept_acts, input.device, input.dtype)
    if ext_backward_func._tc_ok(input):
        # the dense product on this library's tensor-core GEMM (fp32 operands split into tf32 head and tail)
        dim_reduced_input = ext_backward_func.linear_forward(input, rand_matrix.t().contiguous())
    else:
        _lib.note_library_call("input2rp as torch.matmul (fewer than 1024 rows, not fp32 or not CUDA)")
        dim_reduced_input = torch.matmul(input, rand_matrix)
    return dim_reduced_input, rand_matrix


@torch.no_grad()
def rp2input(dim_reduced_input, input_shape, rand_matrix):
    """ops.py:121-125."""
    assert len(dim_reduced_input.size()) == 2
    if ext_backward_func._tc_ok(dim_reduced_input) and rand_matrix.dtype == torch.float32:
        input = ext_backward_func.linear_forward(dim_reduced_input, rand_matrix)   # xq R^T on the tensor cores
    else:
        _lib.note_library_call("rp2input as torch.matmul (fewer than 1024 rows, not fp32 or not CUDA)")
        input = torch.matmul(dim_reduced_input, rand_matrix.t())
    return input.view(input_shape)


def project_and_quantize(input, scheme, rp=True):
    """The (input2rp ->) quantize_activation step shared by qlinear, qspmm_* and QSAGEConv
    (ops.py:142-149, 273-280; layers.py:153-159) -> (quantized, randmat, proj_shape)."""
    if config.kept_frac < 1.0 and rp:
        kept_acts = int(config.kept_frac * input.shape[1] + 0.999)
        if (config.fused_rp and config.compress_activation and not config.simulate and not config.swap
                and input.dim() == 2 and input.is_contiguous()
                and ext_quantization.rp_supported(input.shape[1], kept_acts, input.dtype)):
            # one kernel: projection GEMM (tcgen05) with the statistics + quantise + pack in its epilogue
            with torch.no_grad():
                randmat = _rademacher(input.shape[1], kept_acts, input.device, input.dtype)
                q_bits = config.activation_compression_bits[0]
                q_input, q_scale, q_min = ext_quantization.rp_quantize_pack(input, randmat, q_bits)
            quantized = (q_input, q_bits, q_scale, q_min)
            if config.quantized_hook is not None:
                config.quantized_hook(quantized, randmat)
            return quantized, randmat, torch.Size([input.shape[0], kept_acts])
        dim_reduced_input, randmat = input2rp(input, kept_acts)
    else:
        dim_reduced_input, randmat = input, None
    quantized = quantize_activation(dim_reduced_input, scheme)
    if config.quantized_hook is not None:
        config.quantized_hook(quantized, randmat)
    return quantized, randmat, dim_reduced_input.shape


class qlinear(Function):
    """ops.py:128-178."""

    @staticmethod
    @custom_fwd(device_type="cuda", cast_inputs=torch.float16)
    def forward(ctx, input, weight, bias=None, quantized=None, randmat=None, scheme=None, rp=True):
        if quantized is not None:
            if randmat is None:
                assert rp is False or config.kept_frac == 1.0
                ori_input_shape, proj_input_shape = input.shape, input.shape
            else:
                assert (rp is True and config.kept_frac < 1.0) and (input.shape[1] == randmat.shape[0])
                ori_input_shape, proj_input_shape = input.shape, torch.Size([input.shape[0], randmat.shape[1]])
        else:
            quantized, randmat, proj_input_shape = project_and_quantize(input, scheme, rp)
            ori_input_shape = input.shape
        empty_cache(config.empty_cache_threshold)
        ctx.scheme = scheme
        ctx.saved = quantized, weight, bias, randmat
        ctx.other_args = ori_input_shape, proj_input_shape, rp
        if input.dim() == 2:
            return ext_backward_func.linear_forward(input, weight, bias)
        return F.linear(input, weight, bias)

    @staticmethod
    @custom_bwd(device_type="cuda")
    def backward(ctx, grad_output):
        quantized, weight, bias, randmat = ctx.saved
        ori_input_shape, q_input_shape, rp = ctx.other_args
        del ctx.saved
        grad_input, grad_weight, grad_bias = linear_backward_from_compressed(
            quantized, weight, bias, randmat, ori_input_shape, q_input_shape, rp, grad_output.contiguous(),
            ctx.needs_input_grad[0])
        return grad_input, grad_weight, grad_bias, None, None, None, None


def linear_backward_from_compressed(quantized, weight, bias, randmat, ori_input_shape, q_input_shape, rp,
                                    grad_output, need_grad_input):
    """ops.py:152-178: (grad_input, grad_weight, grad_bias) of y = x W^T + b from the compressed x."""
    projected = config.kept_frac < 1.0 and rp and randmat is not None
    input = None
    if (config.compress_activation and not config.simulate and not config.swap and quantized[1] is not None
            and len(q_input_shape) == 2 and (not projected or config.grad_weight_in_projected_space)
            and ext_backward_func.grad_weight_supported(grad_output, q_input_shape[1], 0, quantized[1])):
        # g^T Xq on the tensor cores with the dequantisation in the operand path: the [N, k] fp32 activation is
        # never written; with a projection, (g^T Xq) R^T instead of g^T (Xq R^T)
        grad_weight, _ = ext_backward_func.grad_weight_from_packed(grad_output, quantized, q_input_shape[1])
        if projected:
            grad_weight = grad_weight.mm(randmat.t())
        else:
            grad_weight = grad_weight.contiguous()
        grad_input = ext_backward_func.linear_forward(grad_output, weight.t()) if need_grad_input else None
        grad_bias = ext_backward_func.rows_scale_colsum(grad_output)[1] if bias is not None else None
        return grad_input, grad_weight, grad_bias
    if (projected and not config.grad_weight_in_projected_space and config.fused_rp and config.compress_activation
            and not config.simulate and not config.swap and len(ori_input_shape) == 2
            and ext_quantization.unpack_rp_supported(ori_input_shape[1], q_input_shape[1])):
        # dequantise + transpose projection in one kernel (reference order: g^T (Xq R^T))
        q_input, q_bits, q_scale, q_min = quantized
        input = ext_quantization.unpack_dequant_rp(q_input, q_bits, q_scale, q_min, q_input_shape[0], randmat)
        projected = False
    if input is None:
        input = dequantize_activation(quantized, q_input_shape)
    del quantized
    empty_cache(config.empty_cache_threshold)
    if projected and config.grad_weight_in_projected_space:
        # grad_W = g^T (Xq R^T) = (g^T Xq) R^T: the [N, D] reconstruction of ops.py:165-166 is never
        # materialised and the large GEMM shrinks from 2*N*out*D to 2*N*out*k flops.
        grad_weight = ext_backward_func.rows_reduce_mm(grad_output, input).mm(randmat.t())
        grad_input = ext_backward_func.linear_forward(grad_output, weight.t()) if need_grad_input else None
        grad_bias = ext_backward_func.rows_scale_colsum(grad_output)[1] if bias is not None else None
    else:
        if projected:
            input = rp2input(input, ori_input_shape, randmat)
        grad_input, grad_weight, grad_bias = ext_backward_func.linear_backward(grad_output, input, weight, bias,
                                                                               need_grad_input)
    del input, grad_output
    empty_cache(config.empty_cache_threshold)
    return grad_input, grad_weight, grad_bias


class qbatch_norm(Function):
    """ops.py:206-254."""

    @staticmethod
    def forward(ctx, input, running_mean, running_var, weight, bias, training, exponential_average_factor,
                eps, scheme):
        quantized = quantize_activation(input, scheme)
        output, save_mean, save_var = ext_backward_func.native_batch_norm(
            input, weight, bias, running_mean, running_var, training, exponential_average_factor, eps)
        ctx.scheme = scheme
        ctx.other_args = input.shape
        ctx.saved = (quantized, weight, running_mean, running_var, save_mean, save_var, training, eps)
        return output

    @staticmethod
    def backward(ctx, grad_output):
        quantized, weight, running_mean, running_var, save_mean, save_var, training, eps = ctx.saved
        q_input_shape = ctx.other_args
        mask = [ctx.needs_input_grad[0], ctx.needs_input_grad[3], ctx.needs_input_grad[4]]
        if (config.compress_activation and not config.simulate and not config.swap and config.bn_backward_from_packed
                and len(q_input_shape) == 2
                and ext_backward_func.batch_norm_backward_from_packed_supported(grad_output, quantized)):
            # both passes of the backward read the packed bytes: no [N, D] reconstruction (ops.py:238)
            del ctx.saved
            grad_input, grad_weight, grad_bias = ext_backward_func.batch_norm_backward_from_packed(
                grad_output, quantized, weight, running_mean, running_var, save_mean, save_var, training, eps, mask)
            return grad_input, None, None, grad_weight, grad_bias, None, None, None, None
        input = dequantize_activation(quantized, q_input_shape)
        del quantized, ctx.saved
        empty_cache(config.empty_cache_threshold)
        grad_input, grad_weight, grad_bias = ext_backward_func.native_batch_norm_backward(
            grad_output.contiguous(), input, weight, running_mean, running_var, save_mean, save_var, training, eps,
            [ctx.needs_input_grad[0], ctx.needs_input_grad[3], ctx.needs_input_grad[4]])
        return grad_input, None, None, grad_weight, grad_bias, None, None, None, None


def _saved_shapes(other, quantized, randmat, scheme):
    """Common forward bookkeeping of qspmm_sum / qspmm_mean (ops.py:263-280, 317-334)."""
    if quantized is not None:
        if randmat is None:
            assert config.kept_frac == 1.0
            return quantized, randmat, other.shape, other.shape
        assert config.kept_frac < 1.0 and (other.shape[1] == randmat.shape[0])
        return quantized, randmat, other.shape, torch.Size([other.shape[0], randmat.shape[1]])
    quantized, randmat, proj_shape = project_and_quantize(other, scheme, True)
    return quantized, randmat, other.shape, proj_shape


class qspmm_sum(Function):
    """ops.py:257-307.  `storage` (optional trailing argument) is the adjacency's SparseStorage; when
    given, the transposed structure for backward comes from its cache."""

    @staticmethod
    @custom_fwd(device_type="cuda", cast_inputs=torch.float16)
    def forward(ctx, row, rowptr, col, value, colptr, csr2csc, has_value, other, quantized=None, randmat=None,
                scheme=None, storage=None):
        result = spmm.spmm_sum_fw(row, rowptr, col, value, colptr, csr2csc, other)
        value_requires_grad = value.requires_grad if has_value else False
        # The compressed copy of `other` is read in backward only by the edge-value gradient.  The
        # reference saves it regardless (ops.py:263-283); with skip_dead_saves it is not produced
        # when nothing will read it.
        if value_requires_grad or not config.skip_dead_saves:
            quantized, randmat, ori_input_shape, proj_input_shape = _saved_shapes(other, quantized, randmat, scheme)
        else:
            quantized, ori_input_shape, proj_input_shape = None, other.shape, other.shape
        empty_cache(config.empty_cache_threshold)
        ctx.saved = row, rowptr, col, value, colptr, csr2csc, quantized, randmat
        ctx.other_args = has_value, ori_input_shape, proj_input_shape, value_requires_grad, other.requires_grad
        ctx.scheme = scheme
        ctx.storage = storage
        return result

    @staticmethod
    @custom_bwd(device_type="cuda")
    def backward(ctx, grad_outputs):
        row, rowptr, col, value, colptr, csr2csc, quantized, randmat = ctx.saved
        has_value, ori_input_shape, q_input_shape, value_requires_grad, mat_requires_grad = ctx.other_args
        # The reference dequantises `other` here unconditionally (ops.py:298-300) although only the
        # edge-value gradient reads it; GCN/SAGE adjacency values never require grad, so it is skipped.
        other = None
        if value_requires_grad:
            other = dequantize_activation(quantized, q_input_shape)
            if config.kept_frac < 1.0:
                other = rp2input(other, ori_input_shape, randmat)
        del quantized, ctx.saved
        transposed = ctx.storage.transposed("sum") if (ctx.storage is not None and mat_requires_grad) else None
        grad_value, grad_mat = spmm.spmm_sum_bw(row, rowptr, col, value, colptr, csr2csc, other,
                                                grad_outputs.contiguous(), has_value, value_requires_grad,
                                                mat_requires_grad, transposed=transposed)
        empty_cache(config.empty_cache_threshold)
        return None, None, None, grad_value, None, None, None, grad_mat, None, None, None, None


class qspmm_mean(Function):
    """ops.py:310-371."""

    @staticmethod
    @custom_fwd(device_type="cuda", cast_inputs=torch.float16)
    def forward(ctx, row, rowptr, col, value, rowcount, colptr, csr2csc, has_value, other, quantized=None,
                randmat=None, scheme=None, storage=None):
        result = spmm.spmm_mean_fw(row, rowptr, col, value, rowcount, colptr, csr2csc, other)
        value_requires_grad = value.requires_grad if has_value else False
        # The compressed copy of `other` is read in backward only by the edge-value gradient.  The
        # reference saves it regardless (ops.py:263-283); with skip_dead_saves it is not produced
        # when nothing will read it.
        if value_requires_grad or not config.skip_dead_saves:
            quantized, randmat, ori_input_shape, proj_input_shape = _saved_shapes(other, quantized, randmat, scheme)
        else:
            quantized, ori_input_shape, proj_input_shape = None, other.shape, other.shape
        empty_cache(config.empty_cache_threshold)
        ctx.saved = row, rowptr, col, value, rowcount, colptr, csr2csc, quantized, randmat
        ctx.other_args = has_value, ori_input_shape, proj_input_shape, value_requires_grad, other.requires_grad
        ctx.scheme = scheme
        ctx.storage = storage
        return result

    @staticmethod
    @custom_bwd(device_type="cuda")
    def backward(ctx, grad_outputs):
        row, rowptr, col, value, rowcount, colptr, csr2csc, quantized, randmat = ctx.saved
        has_value, ori_input_shape, q_input_shape, value_requires_grad, mat_requires_grad = ctx.other_args
        other = None
        if value_requires_grad:  # ops.py:355-364
            other = dequantize_activation(quantized, q_input_shape)
            if config.kept_frac < 1.0:
                other = rp2input(other, ori_input_shape, randmat)
        del quantized, ctx.saved
        transposed = ctx.storage.transposed("mean") if (ctx.storage is not None and mat_requires_grad) else None
        grad_value, grad_mat = spmm.spmm_mean_bw(row, rowptr, col, value, rowcount, colptr, csr2csc, other,
                                                 grad_outputs.contiguous(), has_value, value_requires_grad,
                                                 mat_requires_grad, transposed=transposed)
        empty_cache(config.empty_cache_threshold)
        return None, None, None, grad_value, None, None, None, None, grad_mat, None, None, None, None


def _minmax_forward(ctx, is_max, rowptr, col, value, has_value, other, quantized, scheme):
    """ops.py:378-391 / 410-423: the dense operand is saved quantised WITHOUT projection
    (quantize_activation(other, scheme)) and dequantised in backward for the gather."""
    fw = spmm.spmm_max_fw if is_max else spmm.spmm_min_fw
    output, arg_out = fw(rowptr, col, value, other)
    if quantized is None:
        quantized = quantize_activation(other, scheme)
    else:
        assert isinstance(quantized, tuple)
    empty_cache(config.empty_cache_threshold)
    ctx.saved = col, value, quantized, arg_out
    ctx.other_args = has_value, other.shape, value.requires_grad if has_value else False, other.requires_grad
    ctx.scheme = scheme
    return output


def _minmax_backward(ctx, grad_outputs):
    """ops.py:393-403 / 425-436."""
    col, value, quantized, arg_out = ctx.saved
    has_value, q_input_shape, value_requires_grad, mat_requires_grad = ctx.other_args
    other = dequantize_activation(quantized, q_input_shape)
    del quantized, ctx.saved
    empty_cache(config.empty_cache_threshold)
    grad_value, grad_mat = spmm.spmm_max_bw(col, value, other, arg_out, grad_outputs.contiguous(), has_value,
                                            value_requires_grad, mat_requires_grad)
    return None, None, grad_value, None, grad_mat, None, None, None


class qspmm_max(Function):
    """ops.py:374-403."""

    @staticmethod
    @custom_fwd(device_type="cuda", cast_inputs=torch.float16)
    def forward(ctx, rowptr, col, value, has_value, other, quantized=None, randmat=None, scheme=None):
        return _minmax_forward(ctx, True, rowptr, col, value, has_value, other, quantized, scheme)

    @staticmethod
    @custom_bwd(device_type="cuda")
    def backward(ctx, grad_outputs):
        return _minmax_backward(ctx, grad_outputs)


class qspmm_min(Function):
    """ops.py:406-436."""

    @staticmethod
    @custom_fwd(device_type="cuda", cast_inputs=torch.float16)
    def forward(ctx, rowptr, col, value, has_value, other, quantized=None, randmat=None, scheme=None):
        return _minmax_forward(ctx, False, rowptr, col, value, has_value, other, quantized, scheme)

    @staticmethod
    @custom_bwd(device_type="cuda")
    def backward(ctx, grad_outputs):
        return _minmax_backward(ctx, grad_outputs)
