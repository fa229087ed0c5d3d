"""Sum, Mean, Var and VarMean autograd Functions over libtb200 (counterparts of
trident/operation/sum.py, mean.py, var.py and var_mean.py)."""

from typing import Any

import torch

from trident_b200 import _lib, util


def _forward(input: torch.Tensor, dim, kind: str, correction=0):
    """One launch; the reference runs one Triton program per output element
    (trident/operation/sum.py:57, mean.py:58, var.py:59, var_mean.py:60)."""
    input = input.contiguous()
    y_size, x_size, y_stride, x_stride = util.size_and_stride(input, dim)
    out_a = torch.empty(y_size, device=input.device, dtype=input.dtype)
    out_b = torch.empty(y_size, device=input.device, dtype=input.dtype) if kind == "var_mean" else None
    util.push_trace("tb200_reduce_fwd")
    _lib.reduce_fwd(out_a, out_b, input, y_size, x_size, y_stride, x_stride, kind, correction)
    util.pop_trace()
    return out_a, out_b


def _backward(grad_a, grad_b, input: torch.Tensor, dim, kind: str, correction=0):
    """(trident/operation/sum.py:79, mean.py:80, var.py:82, var_mean.py:86; the zero fill of
    grad_input done there is not needed)."""
    input = input.contiguous()
    y_size, x_size, y_stride, x_stride = util.size_and_stride(input, dim)
    grad_input = torch.empty_like(input)
    if grad_a is None:  # only the mean output of var_mean received a gradient
        grad_a = torch.zeros(y_size, device=input.device, dtype=input.dtype)
    util.push_trace("tb200_reduce_bwd")
    _lib.reduce_bwd(
        grad_input, grad_a.contiguous(), None if grad_b is None else grad_b.contiguous(), input,
        y_size, x_size, y_stride, x_stride, kind, correction,
    )
    util.pop_trace()
    return grad_input


class Sum(torch.autograd.Function):
    @staticmethod
    def forward(ctx: Any, *args: Any, **kwargs: Any):
        input, dim = args
        util.push_trace("Sum.__forward")
        output, _ = _forward(input, dim, "sum")
        util.pop_trace()
        ctx.save_for_backward(input)
        ctx.dim = dim
        return output

    @staticmethod
    def backward(ctx: Any, *grad_outputs: Any):
        (grad_output,) = grad_outputs
        (input,) = ctx.saved_tensors
        util.push_trace("Sum.__backward")
        grad_input = _backward(grad_output, None, input, ctx.dim, "sum")
        util.pop_trace()
        return grad_input, None


class Mean(torch.autograd.Function):
    @staticmethod
    def forward(ctx: Any, *args: Any, **kwargs: Any):
        input, dim = args
        util.push_trace("Mean.__forward")
        output, _ = _forward(input, dim, "mean")
        util.pop_trace()
        ctx.save_for_backward(input)
        ctx.dim = dim
        return output

    @staticmethod
    def backward(ctx: Any, *grad_outputs: Any):
        (grad_output,) = grad_outputs
        (input,) = ctx.saved_tensors
        util.push_trace("Mean.__backward")
        grad_input = _backward(grad_output, None, input, ctx.dim, "mean")
        util.pop_trace()
        return grad_input, None


class Var(torch.autograd.Function):
    @staticmethod
    def forward(ctx: Any, *args: Any, **kwargs: Any):
        input, dim, correction = args
        util.push_trace("Var.__forward")
        output, _ = _forward(input, dim, "var", correction)
        util.pop_trace()
        ctx.save_for_backward(input)
        ctx.dim = dim
        ctx.correction = correction
        return output

    @staticmethod
    def backward(ctx: Any, *grad_outputs: Any):
        (grad_output,) = grad_outputs
        (input,) = ctx.saved_tensors
        util.push_trace("Var.__backward")
        grad_input = _backward(grad_output, None, input, ctx.dim, "var", ctx.correction)
        util.pop_trace()
        return grad_input, None, None


class VarMean(torch.autograd.Function):
    @staticmethod
    def forward(ctx: Any, *args: Any, **kwargs: Any):
        input, dim, correction = args
        util.push_trace("VarMean.__forward")
        var, mean = _forward(input, dim, "var_mean", correction)
        util.pop_trace()
        ctx.save_for_backward(input)
        ctx.dim = dim
        ctx.correction = correction
        return var, mean

    @staticmethod
    def backward(ctx: Any, *grad_outputs: Any):
        grad_var, grad_mean = grad_outputs
        (input,) = ctx.saved_tensors
        util.push_trace("VarMean.__backward")
        grad_input = _backward(grad_var, grad_mean, input, ctx.dim, "var_mean", ctx.correction)
        util.pop_trace()
        return grad_input, None, None
