"""MaskedSoftmax autograd Function over libtb200 (counterpart of
trident/operation/masked_softmax.py)."""

from typing import Any

import torch

from trident_b200 import _lib, util

# the reference kernel masks where `mask > eps` with this eps (trident/language/constant.py)
_MASK_EPS = 2.220446049250313e-16


def as_byte_mask(mask: torch.Tensor, like: torch.Tensor) -> torch.Tensor:
    """One byte per element of `like`, non-zero where the element is masked out.

    bool and uint8 masks are passed through as they are; any other dtype follows the
    reference's rule `mask > eps` (trident/kernel/masked_softmax.py:73).
    """
    if mask.dtype == torch.bool:
        mask = mask.view(torch.uint8)
    elif mask.dtype != torch.uint8:
        mask = (mask > _MASK_EPS).view(torch.uint8)
    if mask.shape != like.shape:
        mask = mask.expand_as(like)
    return mask


class MaskedSoftmax(torch.autograd.Function):
    @staticmethod
    def forward(ctx: Any, *args: Any, **kwargs: Any):
        input, mask, dim = args

        util.push_trace("MaskedSoftmax.__forward")
        output = MaskedSoftmax.__forward(input, mask, dim)
        util.pop_trace()

        ctx.save_for_backward(output)
        ctx.dim = dim

        return output

    @staticmethod
    def backward(ctx: Any, *grad_outputs: Any):
        (grad_output,) = grad_outputs
        (output,) = ctx.saved_tensors

        util.push_trace("MaskedSoftmax.__backward")
        grad_input = MaskedSoftmax.__backward(grad_output, output, ctx.dim)
        util.pop_trace()

        return grad_input, None, None

    @staticmethod
    def __forward(input: torch.Tensor, mask: torch.Tensor, dim: int):
        input = input.contiguous()
        mask = as_byte_mask(mask, input)
        y_size, x_size, y_stride, x_stride = util.size_and_stride(input, dim)
        _, _, m_y_stride, m_x_stride = util.size_and_stride(mask, dim)
        output = torch.empty_like(input)

        util.push_trace("tb200_softmax_fwd")
        _lib.softmax_fwd(output, input, mask, y_size, x_size, y_stride, x_stride, m_y_stride, m_x_stride)
        util.pop_trace()

        return output

    @staticmethod
    def __backward(grad_output: torch.Tensor, output: torch.Tensor, dim: int):
        grad_output = grad_output.contiguous()
        y_size, x_size, y_stride, x_stride = util.size_and_stride(output, dim)
        grad_input = torch.empty_like(output)

        util.push_trace("tb200_softmax_bwd")
        _lib.softmax_bwd(grad_input, grad_output, output, y_size, x_size, y_stride, x_stride)
        util.pop_trace()

        return grad_input
