"""Linear autograd Function over libtb200 (counterpart of trident/operation/linear.py)."""

from typing import Any

import torch

from trident_b200 import _lib, util


def bias_gradient(grad_output: torch.Tensor) -> torch.Tensor:
    """Column sums of grad_output viewed as [rows, N]: one partial-sum launch and one
    finalize launch instead of the per-column kernel plus torch.sum of
    trident/operation/linear.py:136-154."""
    n_size = grad_output.shape[-1]
    rows = grad_output.numel() // n_size
    grad_bias = torch.empty(n_size, device=grad_output.device, dtype=grad_output.dtype)
    workspace = torch.empty(
        max(_lib.linear_bwd_bias_workspace(rows, n_size), 16), dtype=torch.uint8, device=grad_output.device
    )
    _lib.linear_bwd_bias(grad_bias, grad_output, workspace, rows, n_size)
    return grad_bias


class Linear(torch.autograd.Function):
    @staticmethod
    def forward(ctx: Any, *args: Any, **kwargs: Any):
        input, weight, bias, use_accelerator = args

        util.push_trace("Linear.__forward")
        output = Linear.__forward(input, weight, bias, use_accelerator)
        util.pop_trace()

        ctx.save_for_backward(input, weight, bias)
        ctx.use_accelerator = use_accelerator

        return output

    @staticmethod
    def backward(ctx: Any, *grad_outputs: Any):
        (grad_output,) = grad_outputs
        input, weight, bias = ctx.saved_tensors

        util.push_trace("Linear.__backward")
        grad_input, grad_weight, grad_bias = Linear.__backward(grad_output, input, weight, bias, ctx.use_accelerator)
        util.pop_trace()

        return grad_input, grad_weight, grad_bias, None

    @staticmethod
    def __forward(input, weight, bias, use_accelerator):
        num_batches, m_size, k_size = input.shape
        n_size, _ = weight.shape
        output = torch.empty(num_batches, m_size, n_size, device=input.device, dtype=input.dtype)

        util.push_trace("tb200_linear_fwd")
        _lib.linear_fwd(output, input, weight, None if bias is None else bias.contiguous(), use_accelerator)
        util.pop_trace()

        return output

    @staticmethod
    def __backward(grad_output, input, weight, bias, use_accelerator):
        """Three launches (input, weight, bias gradient); the weight gradient is reduced
        over the batch inside the GEMM, so the [batch, N, K] staging buffer and torch.sum
        of trident/operation/linear.py:87,:132-134 do not exist here."""
        grad_output = grad_output.contiguous()
        grad_input = torch.empty_like(input)
        grad_weight = torch.empty(weight.shape, device=weight.device, dtype=weight.dtype)

        util.push_trace("tb200_linear_bwd_input")
        _lib.linear_bwd_input(grad_input, grad_output, weight, use_accelerator)
        util.pop_trace()

        util.push_trace("tb200_linear_bwd_weight")
        _lib.linear_bwd_weight(grad_weight, grad_output, input, use_accelerator)
        util.pop_trace()

        if bias is not None:
            util.push_trace("tb200_linear_bwd_bias")
            grad_bias = bias_gradient(grad_output)
            util.pop_trace()
        else:
            grad_bias = None

        return grad_input, grad_weight, grad_bias
