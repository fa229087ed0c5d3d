"""Attention autograd Function over libtb200 (counterpart of trident/operation/attention.py)."""

from typing import Any

import torch

from trident_b200 import _lib, util


TILE = 128  # rows per query / key tile of the tensor-core kernels


def _additive_mask(mask, dtype):
    """The mask in the additive form the kernels take: a boolean mask (True = attend, as in
    torch.nn.functional.scaled_dot_product_attention) becomes 0 / -inf in `dtype`."""
    if mask.dtype == torch.bool:
        return torch.zeros(mask.shape, dtype=dtype, device=mask.device).masked_fill_(~mask, float("-inf"))
    return mask


def _pad_rows(t, rows):
    """Zero-pads dimension -2 of a [B,H,S,D] tensor to `rows`."""
    return torch.nn.functional.pad(t, (0, 0, 0, rows - t.shape[-2]))


class Attention(torch.autograd.Function):
    """scaled_dot_product_attention (counterpart of trident/operation/attention.py:23-202).

    Beyond the reference's acceptance set: boolean masks (the reference raises,
    operation/attention.py:44-45; the torch oracle of its tests accepts them), any sequence
    length (the reference wants a power of two, operation/attention.py:31-39), and
    `dropout_p > 0` as dropout on the attention OUTPUT, which is where the reference applies it
    (kernel/attention.py:158-161), with an elementwise mask and its exact gradient (the
    reference draws one mask value per feature column and rebuilds the mask from output > 0 in
    its backward, kernel/attention.py:309-313).
    """

    @staticmethod
    def forward(ctx: Any, *args: Any, **kwargs: Any):
        query, key, value, mask, dropout_p, is_causal, softmax_scale, use_accelerator = args

        if query.dim() != 4 or key.dim() != 4 or value.dim() != 4:
            raise ValueError("The dimension of query, key and value should be 4.")

        if not util.is_pow2(query.shape[-1]) or not util.is_pow2(key.shape[-1]) or not util.is_pow2(value.shape[-1]):
            raise ValueError("Attention supports only for power of 2 size tensors.")

        if mask is not None and is_causal:
            raise ValueError("Error because both attn_mask and is_causal are set.")

        if not 0.0 <= dropout_p < 1.0:
            raise ValueError("dropout_p must be in [0, 1).")

        if query.shape != key.shape or key.shape != value.shape:
            raise ValueError("query, key and value should have the same shape.")

        y_size = query.shape[-2]
        kernel_mask = None if mask is None else _additive_mask(mask, query.dtype)
        # 16-bit inputs whose length is not a multiple of the tile: zero rows are appended so that the
        # tensor-core kernels take them. Appended keys never count: under the causal mask they lie
        # after every real query; otherwise an additive -inf over the appended key columns excludes
        # them. Appended query rows are dropped from the output and carry zero gradient in.
        padded = 0
        if query.dtype != torch.float32 and y_size > TILE and y_size % TILE != 0:
            padded = (y_size + TILE - 1) // TILE * TILE
            query, key, value = (_pad_rows(t, padded) for t in (query, key, value))
            if not is_causal:
                if kernel_mask is None:
                    kernel_mask = torch.zeros((1, 1, 1, padded), dtype=query.dtype, device=query.device)
                else:
                    while kernel_mask.dim() < 4:
                        kernel_mask = kernel_mask.unsqueeze(0)
                    pad_q = padded - y_size if kernel_mask.shape[-2] != 1 else 0
                    kernel_mask = torch.nn.functional.pad(kernel_mask.to(query.dtype), (0, padded - y_size, 0, pad_q))
                kernel_mask[..., y_size:] = float("-inf")

        util.push_trace("Attention.__forward")
        output, log_sum_exp = Attention.__forward(query, key, value, kernel_mask, is_causal, softmax_scale)
        util.pop_trace()

        keep = None
        if dropout_p > 0.0:
            keep = torch.rand_like(output, dtype=torch.float32) >= dropout_p

        ctx.save_for_backward(query, key, value, output, log_sum_exp)
        ctx.mask = mask
        ctx.kernel_mask = kernel_mask
        ctx.keep = keep
        ctx.y_size = y_size
        ctx.padded = padded
        ctx.dropout_p = dropout_p
        ctx.is_causal = is_causal
        ctx.softmax_scale = softmax_scale
        ctx.use_accelerator = use_accelerator

        result = output if keep is None else torch.where(keep, output * (1.0 / (1.0 - dropout_p)), 0.0).to(output.dtype)
        return result[:, :, :y_size] if padded else result

    @staticmethod
    def backward(ctx: Any, *grad_outputs: Any):
        (grad_output,) = grad_outputs
        query, key, value, output, log_sum_exp = ctx.saved_tensors
        if ctx.padded:
            grad_output = _pad_rows(grad_output, ctx.padded)
        if ctx.keep is not None:
            grad_output = torch.where(ctx.keep, grad_output * (1.0 / (1.0 - ctx.dropout_p)), 0.0).to(grad_output.dtype)

        mask = ctx.mask
        want_mask_grad = ctx.needs_input_grad[3] and mask is not None and mask.dtype != torch.bool
        util.push_trace("Attention.__backward")
        grad_query, grad_key, grad_value, grad_mask = Attention.__backward(
            grad_output,
            query,
            key,
            value,
            output,
            log_sum_exp,
            ctx.kernel_mask,
            ctx.softmax_scale,
            ctx.is_causal,
            want_mask_grad,
        )
        util.pop_trace()

        if ctx.padded:
            n = ctx.y_size
            grad_query, grad_key, grad_value = (g[:, :, :n] for g in (grad_query, grad_key, grad_value))
            if grad_mask is not None:
                grad_mask = grad_mask[..., : (n if mask.shape[-2] != 1 else 1), :n]
        if grad_mask is not None:
            if tuple(grad_mask.shape) != tuple(mask.shape):
                grad_mask = grad_mask.sum_to_size(mask.shape)
            grad_mask = grad_mask.to(mask.dtype)

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
            # fold the dense gradient back onto the (possibly broadcast) mask the kernel was given
            grad_mask = dense_grad_mask
            if tuple(kernel_mask.shape) != tuple(dense_grad_mask.shape):
                grad_mask = dense_grad_mask.sum_to_size(kernel_mask.shape)

        return grad_query, grad_key, grad_value, grad_mask
