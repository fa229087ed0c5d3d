"""Attention autograd Function over libtb200 (counterpart of trident/operation/attention.py)."""

from typing import Any

import torch

from trident_b200 import _lib, util


class Attention(torch.autograd.Function):
    @staticmethod
    def forward(ctx: Any, *args: Any, **kwargs: Any):
        query, key, value, mask, dropout_p, is_causal, softmax_scale, use_accelerator = args

        if query.dim() != 4 or key.dim() != 4 or value.dim() != 4:
            raise ValueError("The dimension of query, key and value should be 4.")

        if (
            not util.is_pow2(query.shape[-2])
            or not util.is_pow2(query.shape[-1])
            or not util.is_pow2(key.shape[-2])
            or not util.is_pow2(key.shape[-1])
            or not util.is_pow2(value.shape[-2])
            or not util.is_pow2(value.shape[-1])
        ):
            raise ValueError("Attention supports only for power of 2 size tensors.")

        if mask is not None:
            if is_causal:
                raise ValueError("Error because both attn_mask and is_causal are set.")
            if mask.dtype == torch.bool:
                raise ValueError("Boolean mask is not supported yet.")

        if dropout_p != 0.0:
            raise ValueError("Attention dropout is not supported: dropout_p must be 0.")

        if query.shape != key.shape or key.shape != value.shape:
            raise ValueError("query, key and value should have the same shape.")

        util.push_trace("Attention.__forward")
        output, log_sum_exp = Attention.__forward(query, key, value, mask, is_causal, softmax_scale)
        util.pop_trace()

        ctx.save_for_backward(query, key, value, output, log_sum_exp)
        ctx.mask = mask
        ctx.dropout_p = dropout_p
        ctx.is_causal = is_causal
        ctx.softmax_scale = softmax_scale
        ctx.use_accelerator = use_accelerator

        return output

    @staticmethod
    def backward(ctx: Any, *grad_outputs: Any):
        (grad_output,) = grad_outputs
        query, key, value, output, log_sum_exp = ctx.saved_tensors

        util.push_trace("Attention.__backward")
        grad_query, grad_key, grad_value, grad_mask = Attention.__backward(
            grad_output,
            query,
            key,
            value,
            output,
            log_sum_exp,
            ctx.mask,
            ctx.softmax_scale,
            ctx.is_causal,
            ctx.needs_input_grad[3],
        )
        util.pop_trace()

        return grad_query, grad_key, grad_value, grad_mask, None, None, None, None

    @staticmethod
    def __forward(query, key, value, mask, is_causal, softmax_scale):
        """One launch writes the output and the float32 log-sum-exp of every score row
        (the launch site it stands in for is trident/operation/attention.py:109)."""
        assert key.shape[-1] in {16, 32, 64, 128}
        num_batches, num_heads, y_size, x_size = query.shape
        if mask is not None:
            if mask.dtype != query.dtype:
                mask = mask.to(query.dtype)
            while mask.dim() < 4:
                mask = mask.unsqueeze(0)
        output = torch.empty((num_batches, num_heads, y_size, x_size), device=query.device, dtype=query.dtype)
        log_sum_exp = torch.empty(num_batches, num_heads, y_size, device=query.device, dtype=torch.float32)

        util.push_trace("tb200_attention_fwd")
        _lib.attention_fwd(output, log_sum_exp, query, key, value, mask, is_causal, softmax_scale)
        util.pop_trace()

        return output, log_sum_exp

    @staticmethod
    def __backward(grad_output, query, key, value, output, log_sum_exp, mask, softmax_scale, is_causal, want_mask_grad):
        """delta, dq, dk, dv (and the mask gradient only when autograd asks for it; the
        reference allocates it whenever a mask is given, trident/operation/attention.py:154)."""
        num_batches, num_heads, y_size, x_size = query.shape
        grad_output = grad_output.contiguous()
        grad_query = torch.empty((num_batches, num_heads, y_size, x_size), device=query.device, dtype=query.dtype)
        grad_key = torch.empty_like(grad_query)
        grad_value = torch.empty_like(grad_query)
        kernel_mask = mask
        if mask is not None:
            if mask.dtype != query.dtype:
                kernel_mask = mask.to(query.dtype)
            while kernel_mask.dim() < 4:
                kernel_mask = kernel_mask.unsqueeze(0)
        dense_grad_mask = None
        if mask is not None and want_mask_grad:
            dense_grad_mask = torch.empty(
                (num_batches, num_heads, y_size, y_size), device=query.device, dtype=query.dtype
            )
        workspace = torch.empty(
            max(_lib.attention_bwd_workspace(num_batches, num_heads, y_size, x_size, query.dtype), 16),
            dtype=torch.uint8,
            device=query.device,
        )

        util.push_trace("tb200_attention_bwd")
        _lib.attention_bwd(
            grad_query,
            grad_key,
            grad_value,
            dense_grad_mask,
            grad_output,
            query,
            key,
            value,
            output,
            log_sum_exp,
            kernel_mask,
            workspace,
            is_causal,
            softmax_scale,
        )
        util.pop_trace()

        grad_mask = None
        if dense_grad_mask is not None:
            # fold the dense gradient back onto a broadcast mask
            grad_mask = dense_grad_mask
            if tuple(mask.shape) != tuple(dense_grad_mask.shape):
                grad_mask = dense_grad_mask.sum_to_size(mask.shape)
            grad_mask = grad_mask.to(mask.dtype)

        return grad_query, grad_key, grad_value, grad_mask
