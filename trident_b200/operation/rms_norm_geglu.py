"""RMSNorm followed by GEGLU as one autograd Function (no counterpart in the reference, which
runs trident/function/function.py:202-208 and :70-80 back to back).

Forward: one pass over x for the row statistic rms, then ONE tensor-core GEMM on the raw x whose
epilogue multiplies each accumulator row by 1 / (rms + eps): with the norm weight folded into the
projection weight, W' = W * diag(w_norm), this is GEGLU(RMSNorm(x)) and the normalised copy of x
is neither written nor read (2 * rows * cols elements of traffic less). Backward: the normalised
x is recomputed by the RMSNorm forward kernel and the two operations' own backward kernels run in
turn, so the gradients are those of the unfused chain.

The folded weight costs one elementwise pass over W per call unless the caller passes a
`folded_weight` computed once (inference, or any stretch over which W and w_norm are fixed).
"""

from typing import Any

import torch

from trident_b200 import _lib, config, util
from trident_b200.operation.geglu import GEGLU
from trident_b200.operation.rms_norm import RMSNorm


class RMSNormGEGLU(torch.autograd.Function):
    @staticmethod
    def forward(ctx: Any, *args: Any, **kwargs: Any):
        input, p, norm_weight, weight, bias, eps, folded_weight = args
        if input.dim() != 2:
            raise ValueError("rms_norm_geglu takes a 2-D input [rows, features].")
        y_size, x_size = input.shape
        n_size = weight.shape[0]
        if n_size % 2 != 0:
            raise ValueError(f"GEGLU needs an even number of output features, got {n_size}.")
        partial_size = x_size if p < 0.0 or p > 1.0 else int(x_size * p)
        if partial_size <= 0:
            raise ValueError(f"p={p} selects an empty slice of {x_size} features.")
        norm_weight = norm_weight.contiguous()

        util.push_trace("RMSNormGEGLU.__forward")
        rms = torch.empty(y_size, device=input.device, dtype=torch.float32)
        # y = null: the row statistic alone
        _lib.rms_norm_fwd(None, rms, input, norm_weight, None, y_size, x_size, input.stride(0), input.stride(1),
                          partial_size, eps)
        row_scale = torch.reciprocal(rms + eps)
        folded = folded_weight if folded_weight is not None else (weight * norm_weight).contiguous()
        output = torch.empty(1, y_size, n_size // 2, device=input.device, dtype=input.dtype)
        state_gate = torch.empty(1, y_size, n_size, device=input.device, dtype=input.dtype)
        fused = _lib.geglu_fwd_row_scaled(
            output, state_gate, input.unsqueeze(0), folded, None if bias is None else bias.contiguous(), row_scale,
            config.geglu_tanh_approximation,
        )
        if not fused:
            # inputs the tensor-core GEMM does not take: the two kernels one after the other
            normed = torch.empty_like(input, memory_format=torch.contiguous_format)
            _lib.rms_norm_fwd(normed, rms, input, norm_weight, None, y_size, x_size, input.stride(0),
                              input.stride(1), partial_size, eps)
            _lib.geglu_fwd(output, state_gate, normed.unsqueeze(0), weight,
                           None if bias is None else bias.contiguous(), config.geglu_tanh_approximation, False)
        util.pop_trace()

        ctx.save_for_backward(input, norm_weight, weight, bias, rms, state_gate)
        ctx.partial_size = partial_size
        ctx.p = p
        ctx.eps = eps
        ctx.gelu_tanh = config.geglu_tanh_approximation
        ctx.fused = fused
        return output.view(y_size, n_size // 2)

    @staticmethod
    def backward(ctx: Any, *grad_outputs: Any):
        (grad_output,) = grad_outputs
        input, norm_weight, weight, bias, rms, state_gate = ctx.saved_tensors
        y_size, x_size = input.shape

        util.push_trace("RMSNormGEGLU.__backward")
        # recompute the normalised input (one RMSNorm forward launch) ...
        normed = torch.empty_like(input, memory_format=torch.contiguous_format)
        rms_again = torch.empty_like(rms)
        _lib.rms_norm_fwd(normed, rms_again, input, norm_weight, None, y_size, x_size, input.stride(0),
                          input.stride(1), ctx.partial_size, ctx.eps)
        # ... then GEGLU's backward on it and RMSNorm's backward on the result
        backward_geglu = getattr(GEGLU, "_GEGLU__backward")
        grad_normed, grad_weight, grad_bias = backward_geglu(
            grad_output.reshape(1, y_size, -1), normed.unsqueeze(0), weight, bias, state_gate, False, ctx.gelu_tanh
        )
        backward_norm = getattr(RMSNorm, "_RMSNorm__backward")
        grad_input, grad_norm_weight, _ = backward_norm(
            grad_normed.view(y_size, x_size), input, ctx.p, rms, norm_weight, None, ctx.eps
        )
        util.pop_trace()

        return grad_input, None, grad_norm_weight, grad_weight, grad_bias, None, None
