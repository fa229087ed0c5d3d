"""Torch eager restatement of each operation, exactly as the reference's tests state it.

Every function works on CPU or CUDA tensors of any floating dtype and supports autograd,
so `backward(grad_output)` gives the oracle gradients.
"""

import torch


def layer_norm(input, normalized_shape, weight=None, bias=None, eps=1e-05):
    """tests/test_layer_norm.py:28-47 compares against torch.nn.functional.layer_norm."""
    return torch.nn.functional.layer_norm(input, normalized_shape, weight, bias, eps)


def rms_norm(input, p, weight, bias=None, eps=1e-08):
    """tests/test_rms_norm.py:22-39: eps is added to the RMS (outside the square root) and
    0 <= p <= 1 takes the norm over the leading int(x_size * p) features."""
    x_size = input.shape[-1]
    if p < 0.0 or p > 1.0:
        norm = input.norm(2, dim=-1, keepdim=True)
        partial_size = x_size
    else:
        partial_size = int(x_size * p)
        partial_input, _ = torch.split(input, [partial_size, x_size - partial_size], dim=-1)
        norm = partial_input.norm(2, dim=-1, keepdim=True)
    rms = norm * partial_size ** (-1.0 / 2)
    output = input / (rms + eps)
    if bias is not None:
        return weight * output + bias
    return weight * output


def softmax(input, dim):
    """tests/test_softmax.py:26 compares against torch.nn.functional.softmax."""
    return torch.nn.functional.softmax(input, 0 if dim == 0 else -1)


def masked_softmax(input, mask, dim):
    """tests/test_masked_softmax.py:22-26: masked positions become -inf before softmax."""
    filled = torch.where(mask.bool(), float("-inf"), input)
    return torch.nn.functional.softmax(filled, 0 if dim == 0 else -1)


def sum(input, dim):
    """tests/test_sum.py:22-29 compares against torch.sum."""
    return torch.sum(input, dim)


def mean(input, dim):
    """tests/test_mean.py:22-29 compares against torch.mean."""
    return torch.mean(input, dim)


def var(input, dim, correction=1):
    """tests/test_var.py:22-26 compares against torch.var."""
    return torch.var(input, dim, correction=correction)


def var_mean(input, dim, correction=1):
    """tests/test_var_mean.py compares against torch.var_mean."""
    return torch.var_mean(input, dim, correction=correction)


def linear(input, weight, bias=None):
    """tests/test_linear.py:27-36 compares against torch.nn.functional.linear."""
    return torch.nn.functional.linear(input, weight, bias)


def geglu(input, weight, bias=None):
    """tests/test_geglu.py:22-24: state is the first half of the projection, gate the
    second half, and the oracle's GELU is the exact erf form."""
    state, gate = torch.nn.functional.linear(input, weight, bias).chunk(2, -1)
    return state * torch.nn.functional.gelu(gate)


def scaled_dot_product_attention(query, key, value, attn_mask=None, is_causal=False):
    """tests/test_attention.py:31-39 compares against torch's scaled_dot_product_attention
    (scale 1/sqrt(head size), additive float mask or causal mask)."""
    return torch.nn.functional.scaled_dot_product_attention(
        query, key, value, attn_mask=attn_mask, is_causal=is_causal
    )


def forward_backward(fn, inputs, grad_output):
    """Runs fn(*inputs) and backpropagates grad_output. `inputs` is a list whose tensor
    entries flagged requires_grad receive gradients; returns (output, [grads])."""
    leaves = []
    for v in inputs:
        if isinstance(v, torch.Tensor) and v.is_floating_point() and v.requires_grad:
            leaves.append(v)
    out = fn(*inputs)
    grads = torch.autograd.grad(out, leaves, grad_output) if leaves else ()
    return out.detach(), [g.detach() for g in grads]
