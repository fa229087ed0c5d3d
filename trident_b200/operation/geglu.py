"""GEGLU autograd Function over libtb200 (counterpart of trident/operation/geglu.py)."""

from typing import Any

import torch

from trident_b200 import _lib, config, util


class GEGLU(torch.autograd.Function):
    @staticmethod
    def forward(ctx: Any, *args: Any, **kwargs: Any):
        input, weight, bias, use_accelerator = args

        util.push_trace("GEGLU.__forward")
        output, state_gate = GEGLU.__forward(input, weight, bias, use_accelerator)
        util.pop_trace()

        ctx.save_for_backward(input, weight, bias, state_gate)
        # the reference's backward never enables TF32 (trident/operation/geglu.py:33)
        ctx.use_accelerator = False
        ctx.gelu_tanh = config.geglu_tanh_approximation

        return output

    @staticmethod
    def backward(ctx: Any, *grad_outputs: Any):
        (grad_output,) = grad_outputs
        input, weight, bias, state_gate = ctx.saved_tensors

        util.push_trace("GEGLU.__backward")
        grad_input, grad_weight, grad_bias = GEGLU.__backward(
            grad_output, input, weight, bias, state_gate, ctx.use_accelerator, ctx.gelu_tanh
        )
        util.pop_trace()

        return grad_input, grad_weight, grad_bias, None

    @staticmethod
    def __forward(input, weight, bias, use_accelerator):
        """One launch computes state_gate = x w^T + b and out = state * gelu(gate)
        (the launch site it stands in for is trident/operation/geglu.py:65)."""
        num_batches, m_size, k_size = input.shape
        n_size, _ = weight.shape
        if n_size % 2 != 0:
            raise ValueError(f"GEGLU needs an even number of output features, got {n_size}.")
        x_size = n_size // 2
        output = torch.empty(num_batches, m_size, x_size, device=input.device, dtype=input.dtype)
        state_gate = torch.empty(num_batches, m_size, n_size, device=input.device, dtype=input.dtype)

        util.push_trace("tb200_geglu_fwd")
        _lib.geglu_fwd(
            output,
            state_gate,
            input,
            weight,
            None if bias is None else bias.contiguous(),
            config.geglu_tanh_approximation,
            use_accelerator,
        )
        util.pop_trace()

        return output, state_gate

    @staticmethod
    def __backward(grad_output, input, weight, bias, state_gate, use_accelerator, gelu_tanh):
        """d_state_gate elementwise, then the Linear backward GEMMs on it
        (trident/operation/geglu.py:100-178 without its staging buffers)."""
        num_batches, m_size, n_size = state_gate.shape
        grad_output = grad_output.contiguous()
        grad_state_gate = torch.empty_like(state_gate)
        grad_input = torch.empty_like(input)
        grad_weight = torch.empty(weight.shape, device=weight.device, dtype=weight.dtype)

        rows = num_batches * m_size
        grad_bias = None
        if bias is not None:
            # the bias gradient (column sums of d_state_gate) is taken in the same pass
            util.push_trace("tb200_geglu_bwd_elementwise_bias")
            grad_bias = torch.empty(n_size, device=state_gate.device, dtype=state_gate.dtype)
            workspace = torch.empty(
                max(_lib.linear_bwd_bias_workspace(rows, n_size), 16), dtype=torch.uint8, device=state_gate.device
            )
            _lib.geglu_bwd_elementwise_bias(
                grad_state_gate, grad_bias, grad_output, state_gate, workspace, rows, n_size, gelu_tanh
            )
            util.pop_trace()
        else:
            util.push_trace("tb200_geglu_bwd_elementwise")
            _lib.geglu_bwd_elementwise(grad_state_gate, grad_output, state_gate, rows, n_size, gelu_tanh)
            util.pop_trace()

        util.push_trace("tb200_linear_bwd_input")
        _lib.linear_bwd_input(grad_input, grad_state_gate, weight, use_accelerator)
        util.pop_trace()

        util.push_trace("tb200_linear_bwd_weight")
        _lib.linear_bwd_weight(grad_weight, grad_state_gate, input, use_accelerator)
        util.pop_trace()

        return grad_input, grad_weight, grad_bias
