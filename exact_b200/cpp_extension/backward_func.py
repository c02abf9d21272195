"""Stand-in for the reference's `exact.cpp_extension.backward_func` module
(exact/exact/cpp_extension/backward_func.cc:83-107): library GEMMs and ATen batch-norm pass-throughs,
kept as library calls exactly as the reference keeps them."""
import torch


def linear_backward(grad_output, input, weight, bias=None, need_grad_input=True):
    """backward_func.cc:83-93.  The input gradient is left out (None) when the caller has no use for it."""
    grad_input = grad_output.mm(weight) if need_grad_input else None
    grad_weight = grad_output.t().mm(input)
    grad_bias = grad_output.sum(0) if bias is not None else None
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
