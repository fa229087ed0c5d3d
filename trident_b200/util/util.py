"""Host-side helpers of the operation layer; counterparts of trident/util/util.py."""

import torch

from trident_b200 import config

__all__ = [
    "calculate_fan_in_and_fan_out",
    "fill",
    "is_pow2",
    "size_and_stride",
    "push_trace",
    "pop_trace",
    "uniform",
    "zero",
]


def calculate_fan_in_and_fan_out(input: torch.Tensor):
    with torch.no_grad():
        return torch.nn.init._calculate_fan_in_and_fan_out(input)


def fill(inp, val):
    with torch.no_grad():
        return inp.fill_(val)


def is_pow2(value):
    """True for 1, 2, 4, ... (trident/util/util.py:61-62)."""
    return value != 0 and (value & (value - 1)) == 0


def size_and_stride(input: torch.Tensor, dim: int):
    """(rows, cols, row_stride, col_stride) of a 2-D tensor reduced along `dim`.

    dim == 0 reduces down the columns, every other value along the last dimension
    (trident/util/util.py:65-77). Only 2-D inputs are accepted: the reference's 3-D
    branch returns six values that none of its row operations can unpack.
    """
    if input.dim() != 2:
        raise ValueError(f"{dim} is not supported.")
    if dim == 0:
        x_size, y_size = input.shape
        return y_size, x_size, input.stride(1), input.stride(0)
    y_size, x_size = input.shape
    return y_size, x_size, input.stride(0), input.stride(1)


def push_trace(message: str):
    """Opens an NVTX range when config.use_trace is set (trident/util/util.py:93-95)."""
    if config.use_trace and torch.cuda.is_available():
        torch.cuda.nvtx.range_push(message)


def pop_trace():
    if config.use_trace and torch.cuda.is_available():
        torch.cuda.nvtx.range_pop()


def uniform(input: torch.Tensor, a: float = 0.0, b: float = 1.0):
    with torch.no_grad():
        return torch.nn.init.uniform_(input, a, b)


def zero(inp):
    with torch.no_grad():
        return inp.zero_()
