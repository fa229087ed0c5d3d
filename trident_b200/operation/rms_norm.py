"""RMSNorm autograd Function over libtb200 (counterpart of trident/operation/rms_norm.py)."""

from typing import Any

import torch

from trident_b200 import _lib, util


def partial_size(x_size: int, p: float) -> int:
    """Width of the leading slice the RMS is taken over: all of it unless 0 <= p <= 1
    (trident/operation/rms_norm.py:68; int(x_size * p) as in tests/test_rms_norm.py:29)."""
    return x_size if p < 0.0 or p > 1.0 else int(x_size * p)


class RMSNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx: Any, *args: Any, **kwargs: Any):
        input, p, weight, bias, eps = args

        util.push_trace("RMSNorm.__forward")
        output, rms = RMSNorm.__forward(input, p, weight, bias, eps)
        util.pop_trace()

        ctx.save_for_backward(input, rms, weight, bias)
        ctx.p = p
        ctx.eps = eps

        return output

    @staticmethod
    def backward(ctx: Any, *grad_outputs: Any):
        (grad_output,) = grad_outputs
        input, rms, weight, bias = ctx.saved_tensors

        util.push_trace("RMSNorm.__backward")
        grad_input, grad_weight, grad_bias = RMSNorm.__backward(
            grad_output, input, ctx.p, rms, weight, bias, ctx.eps
        )
        util.pop_trace()

        return grad_input, None, grad_weight, grad_bias, None

    @staticmethod
    def __forward(input: torch.Tensor, p: float, weight: torch.Tensor, bias: torch.Tensor, eps: float):
        y_size, x_size, y_stride, x_stride = util.size_and_stride(input, 1)
        partial = partial_size(x_size, p)
        if partial <= 0:
            raise ValueError(f"p={p} selects an empty slice of {x_size} features.")
        output = torch.empty((y_size, x_size), device=input.device, dtype=input.dtype)
        rms = torch.empty(y_size, device=input.device, dtype=torch.float32)

        util.push_trace("tb200_rms_norm_fwd")
        _lib.rms_norm_fwd(
            output,
            rms,
            input,
            weight.contiguous(),
            None if bias is None else bias.contiguous(),
            y_size,
            x_size,
            y_stride,
            x_stride,
            partial,
            eps,
        )
        util.pop_trace()

        return output, rms

    @staticmethod
    def __backward(grad_output, input, p, rms, weight, bias, eps):
        """dx, dw (and db) in one pass; stands in for the launch at
        trident/operation/rms_norm.py:98, the torch.sum at :117 and the Sum kernel at :122."""
        y_size, x_size, y_stride, x_stride = util.size_and_stride(input, 1)
        grad_output = grad_output.contiguous()
        grad_input = torch.empty((y_size, x_size), device=input.device, dtype=input.dtype)
        grad_weight = torch.empty_like(weight)
        grad_bias = torch.empty_like(bias) if bias is not None else None
        workspace = torch.empty(
            max(_lib.rms_norm_bwd_workspace(y_size, x_size), 16), dtype=torch.uint8, device=input.device
        )

        util.push_trace("tb200_rms_norm_bwd")
        _lib.rms_norm_bwd(
            grad_input,
            grad_weight,
            grad_bias,
            grad_output,
            input,
            weight.contiguous(),
            rms,
            workspace,
            y_size,
            x_size,
            y_stride,
            x_stride,
            partial_size(x_size, p),
            eps,
        )
        util.pop_trace()

        return grad_input, grad_weight, grad_bias
