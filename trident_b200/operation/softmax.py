"""Softmax autograd Function over libtb200 (counterpart of trident/operation/softmax.py)."""

from typing import Any

import torch

from trident_b200 import _lib, util


class Softmax(torch.autograd.Function):
    @staticmethod
    def forward(ctx: Any, *args: Any, **kwargs: Any):
        input, dim = args

        util.push_trace("Softmax.__forward")
        output = Softmax.__forward(input, dim)
        util.pop_trace()

        ctx.save_for_backward(output)
        ctx.dim = dim

        return output

    @staticmethod
    def backward(ctx: Any, *grad_outputs: Any):
        (grad_output,) = grad_outputs
        (output,) = ctx.saved_tensors

        util.push_trace("Softmax.__backward")
        grad_input = Softmax.__backward(grad_output, output, ctx.dim)
        util.pop_trace()

        return grad_input, None

    @staticmethod
    def __forward(input: torch.Tensor, dim: int):
        input = input.contiguous()
        y_size, x_size, y_stride, x_stride = util.size_and_stride(input, dim)
        output = torch.empty_like(input)

        util.push_trace("tb200_softmax_fwd")
        _lib.softmax_fwd(output, input, None, y_size, x_size, y_stride, x_stride)
        util.pop_trace()

        return output

    @staticmethod
    def __backward(grad_output: torch.Tensor, output: torch.Tensor, dim: int):
        """delta and dx in one launch (trident/operation/softmax.py:81 and :97 are two)."""
        grad_output = grad_output.contiguous()
        y_size, x_size, y_stride, x_stride = util.size_and_stride(output, dim)
        grad_input = torch.empty_like(output)

        util.push_trace("tb200_softmax_bwd")
        _lib.softmax_bwd(grad_input, grad_output, output, y_size, x_size, y_stride, x_stride)
        util.pop_trace()

        return grad_input
