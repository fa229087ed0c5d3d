"""LayerNorm autograd Function over libtb200 (counterpart of trident/operation/layer_norm.py)."""

import math
from typing import Any

import torch

from trident_b200 import _lib, util


def _workspace(nbytes, device):
    return torch.empty(max(int(nbytes), 16), dtype=torch.uint8, device=device)


class LayerNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx: Any, *args: Any, **kwargs: Any):
        input, normalized_shape, weight, bias, eps = args

        util.push_trace("LayerNorm.__forward")
        output, rstd, mean = LayerNorm.__forward(input, normalized_shape, weight, bias, eps)
        util.pop_trace()

        ctx.save_for_backward(input, weight, bias, rstd, mean)
        ctx.normalized_shape = normalized_shape

        return output

    @staticmethod
    def backward(ctx: Any, *grad_outputs: Any):
        (grad_output,) = grad_outputs
        input, weight, bias, rstd, mean = ctx.saved_tensors

        util.push_trace("LayerNorm.__backward")
        grad_input, grad_weight, grad_bias = LayerNorm.__backward(
            grad_output, input, ctx.normalized_shape, weight, bias, rstd, mean
        )
        util.pop_trace()

        return grad_input, None, grad_weight, grad_bias, None

    @staticmethod
    def __forward(input, normalized_shape, weight, bias, eps):
        """One launch: y plus float32 mean and rstd per row
        (the launch site it stands in for is trident/operation/layer_norm.py:64)."""
        x_size = math.prod(normalized_shape)
        y_size = input.numel() // x_size
        input = input.contiguous()
        output = torch.empty_like(input)
        rstd = torch.empty(y_size, device=input.device, dtype=torch.float32)
        mean = torch.empty(y_size, device=input.device, dtype=torch.float32)

        util.push_trace("tb200_layer_norm_fwd")
        _lib.layer_norm_fwd(
            output,
            mean,
            rstd,
            input,
            None if weight is None else weight.contiguous(),
            None if bias is None else bias.contiguous(),
            y_size,
            x_size,
            eps,
        )
        util.pop_trace()

        return output, rstd, mean

    @staticmethod
    def __backward(grad_output, input, normalized_shape, weight, bias, rstd, mean):
        """dx, dw and db from one pass over (x, dy); the per-row weight-gradient staging
        buffer and the torch.sum calls of trident/operation/layer_norm.py:88-122 are
        replaced by per-CTA column partials inside the library's workspace."""
        x_size = math.prod(normalized_shape)
        y_size = grad_output.numel() // x_size
        input = input.contiguous()
        grad_output = grad_output.contiguous()
        grad_input = torch.empty_like(input)
        grad_weight = torch.empty_like(weight) if weight is not None else None
        grad_bias = torch.empty_like(bias) if bias is not None else None
        workspace = None
        if grad_weight is not None or grad_bias is not None:
            workspace = _workspace(_lib.layer_norm_bwd_workspace(y_size, x_size), input.device)

        util.push_trace("tb200_layer_norm_bwd")
        _lib.layer_norm_bwd(
            grad_input,
            grad_weight,
            grad_bias,
            grad_output,
            input,
            None if weight is None else weight.contiguous(),
            mean,
            rstd,
            workspace,
            y_size,
            x_size,
        )
        util.pop_trace()

        return grad_input, grad_weight, grad_bias
