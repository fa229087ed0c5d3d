"""ctypes binding of libtb200.so, the C-ABI kernel library declared in include/tb200.h.

Every wrapper takes torch CUDA tensors, passes raw device pointers, element strides and
the current CUDA stream, and raises on a non-zero status. There is no CPU or PyTorch
fallback: without the built library, or without a CUDA device, the calls fail loudly.
"""

import ctypes
import os

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("TB200_LIB", os.path.join(_HERE, "libtb200.so"))

_DTYPE = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}

c_i64 = ctypes.c_int64
c_int = ctypes.c_int
c_f32 = ctypes.c_float
c_ptr = ctypes.c_void_p
c_size = ctypes.c_size_t

# name -> (restype, argtypes); mirrors include/tb200.h one to one.
SIGNATURES = {
    "tb200_last_error": (ctypes.c_char_p, []),
    "tb200_version": (c_int, []),
    "tb200_device_check": (c_int, [c_int]),
    "tb200_last_kernel": (ctypes.c_char_p, []),
    "tb200_last_launch_count": (c_int, []),
    "tb200_set_norm_fused_finalize": (c_int, [c_int]),
    "tb200_test_wait_fault": (c_int, [c_int]),
    "tb200_total_launches": (c_i64, []),
    "tb200_device_status": (c_int, [c_int]),
    "tb200_layer_norm_fwd": (c_int, [c_ptr] * 6 + [c_i64, c_i64, c_f32, c_int, c_ptr]),
    "tb200_layer_norm_bwd_workspace": (c_size, [c_i64, c_i64]),
    "tb200_layer_norm_bwd": (c_int, [c_ptr] * 9 + [c_size, c_i64, c_i64, c_int, c_ptr]),
    "tb200_layer_norm_bwd_static": (c_int, [c_ptr] * 8 + [c_i64, c_i64, c_int, c_ptr]),
    "tb200_rms_norm_fwd": (c_int, [c_ptr] * 5 + [c_i64] * 5 + [c_f32, c_int, c_ptr]),
    "tb200_rms_norm_bwd_workspace": (c_size, [c_i64, c_i64]),
    "tb200_rms_norm_bwd": (c_int, [c_ptr] * 8 + [c_size] + [c_i64] * 5 + [c_f32, c_int, c_ptr]),
    "tb200_reduce_fwd": (c_int, [c_ptr] * 3 + [c_i64] * 4 + [c_int, c_f32, c_int, c_ptr]),
    "tb200_reduce_bwd": (c_int, [c_ptr] * 4 + [c_i64] * 4 + [c_int, c_f32, c_int, c_ptr]),
    "tb200_softmax_fwd": (c_int, [c_ptr] * 3 + [c_i64] * 6 + [c_int, c_ptr]),
    "tb200_softmax_bwd": (c_int, [c_ptr] * 3 + [c_i64] * 4 + [c_int, c_ptr]),
    "tb200_linear_fwd": (c_int, [c_ptr] * 4 + [c_i64] * 9 + [c_int, c_int, c_ptr]),
    "tb200_linear_bwd_input": (c_int, [c_ptr] * 3 + [c_i64] * 9 + [c_int, c_int, c_ptr]),
    "tb200_linear_bwd_weight": (c_int, [c_ptr] * 3 + [c_i64] * 7 + [c_int, c_int, c_ptr]),
    "tb200_linear_bwd_bias_workspace": (c_size, [c_i64, c_i64]),
    "tb200_linear_bwd_bias": (c_int, [c_ptr] * 3 + [c_size, c_i64, c_i64, c_int, c_ptr]),
    "tb200_geglu_fwd": (c_int, [c_ptr] * 5 + [c_i64] * 9 + [c_int, c_int, c_int, c_ptr]),
    "tb200_geglu_fwd_row_scaled": (c_int, [c_ptr] * 6 + [c_i64] * 9 + [c_int, c_int, c_ptr]),
    "tb200_geglu_bwd_elementwise": (c_int, [c_ptr] * 3 + [c_i64, c_i64, c_int, c_int, c_ptr]),
    "tb200_geglu_bwd_elementwise_bias": (c_int, [c_ptr] * 5 + [c_size, c_i64, c_i64, c_int, c_int, c_ptr]),
    "tb200_attention_fwd": (
        c_int,
        [c_ptr] * 6 + [c_i64] * 4 + [c_ptr] * 5 + [c_int, c_f32, c_int, c_ptr],
    ),
    "tb200_attention_bwd_workspace": (c_size, [c_i64] * 4 + [c_int]),
    "tb200_attention_bwd": (
        c_int,
        [c_ptr] * 12 + [c_size] + [c_i64] * 4 + [c_ptr] * 5 + [c_int, c_f32, c_int, c_ptr],
    ),
}

_lib = None


class Tb200Error(RuntimeError):
    """A libtb200 call was rejected (negative status) or its launch failed (positive)."""


def load():
    """Loads libtb200.so once and declares every prototype; raises if it is missing."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise Tb200Error(
                f"{LIB_PATH} is missing: build it with `python -m trident_b200.build` "
                "(there is no fallback implementation)"
            )
        lib = ctypes.CDLL(LIB_PATH)
        for name, (restype, argtypes) in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype = restype
            fn.argtypes = argtypes
        _lib = lib
    return _lib


def last_error():
    return load().tb200_last_error().decode()


def last_kernel():
    return load().tb200_last_kernel().decode()


def last_launch_count():
    return load().tb200_last_launch_count()


def total_launches():
    """Kernels launched by the library in this process so far."""
    return load().tb200_total_launches()


def device_status(reset=False):
    """Synchronises and returns the tensor-core kernels' status word (0 = healthy)."""
    return load().tb200_device_status(1 if reset else 0)


def set_norm_fused_finalize(on):
    """Norm backward: fold the weight/bias gradient inside the main launch (default) or in a
    second kernel. Returns the old setting."""
    return load().tb200_set_norm_fused_finalize(1 if on else 0)


def test_wait_fault(mode):
    """Test hook (calling thread): 1 makes one bounded wait of the next attention forward launches
    run out (see include/tb200.h); 0 restores normal operation. Returns the old mode."""
    return load().tb200_test_wait_fault(int(mode))


test_wait_fault.__test__ = False  # not a pytest test


def dtype_code(dtype):
    try:
        return _DTYPE[dtype]
    except KeyError:
        raise ValueError(f"Unable to convert the given input: '{dtype}'.") from None


def _check(status, what):
    if status != 0:
        raise Tb200Error(f"{what} failed with status {status}: {last_error()}")


def _ptr(t):
    return None if t is None else t.data_ptr()


def _stream(t):
    return torch.cuda.current_stream(t.device).cuda_stream


def _require_cuda(*tensors):
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise Tb200Error("trident_b200 kernels run on CUDA tensors only (no CPU fallback)")


def _strides4(t):
    return (c_i64 * 4)(*t.stride())


# --------------------------------------------------------------------------- row ops
def layer_norm_fwd(y, mean, rstd, x, weight, bias, rows, cols, eps):
    _require_cuda(y, x, weight, bias)
    _check(
        load().tb200_layer_norm_fwd(
            _ptr(y), _ptr(mean), _ptr(rstd), _ptr(x), _ptr(weight), _ptr(bias),
            rows, cols, eps, dtype_code(x.dtype), _stream(x),
        ),
        "tb200_layer_norm_fwd",
    )


def layer_norm_bwd_workspace(rows, cols):
    return load().tb200_layer_norm_bwd_workspace(rows, cols)


def layer_norm_bwd(dx, dweight, dbias, dy, x, weight, mean, rstd, workspace, rows, cols):
    _require_cuda(dx, dy, x)
    _check(
        load().tb200_layer_norm_bwd(
            _ptr(dx), _ptr(dweight), _ptr(dbias), _ptr(dy), _ptr(x), _ptr(weight),
            _ptr(mean), _ptr(rstd), _ptr(workspace),
            0 if workspace is None else workspace.numel() * workspace.element_size(),
            rows, cols, dtype_code(x.dtype), _stream(x),
        ),
        "tb200_layer_norm_bwd",
    )


def layer_norm_bwd_static(dx, dweight, dbias, dy, x, weight, mean, rstd, rows, cols):
    """LayerNorm backward for callers that cannot allocate device memory: same outputs as
    layer_norm_bwd, no workspace argument (the library's built-in 2 MiB scratch is used;
    cols <= 8192; calls on one device must not overlap on the GPU)."""
    _require_cuda(dx, dy, x)
    _check(
        load().tb200_layer_norm_bwd_static(
            _ptr(dx), _ptr(dweight), _ptr(dbias), _ptr(dy), _ptr(x), _ptr(weight),
            _ptr(mean), _ptr(rstd), rows, cols, dtype_code(x.dtype), _stream(x),
        ),
        "tb200_layer_norm_bwd_static",
    )


def rms_norm_fwd(y, rms, x, weight, bias, rows, cols, row_stride, col_stride, partial, eps):
    _require_cuda(y, x, weight, bias)
    _check(
        load().tb200_rms_norm_fwd(
            _ptr(y), _ptr(rms), _ptr(x), _ptr(weight), _ptr(bias),
            rows, cols, row_stride, col_stride, partial, eps, dtype_code(x.dtype), _stream(x),
        ),
        "tb200_rms_norm_fwd",
    )


def rms_norm_bwd_workspace(rows, cols):
    return load().tb200_rms_norm_bwd_workspace(rows, cols)


def rms_norm_bwd(dx, dweight, dbias, dy, x, weight, rms, workspace, rows, cols, row_stride,
                 col_stride, partial, eps):
    _require_cuda(dx, dy, x, weight)
    _check(
        load().tb200_rms_norm_bwd(
            _ptr(dx), _ptr(dweight), _ptr(dbias), _ptr(dy), _ptr(x), _ptr(weight), _ptr(rms),
            _ptr(workspace), workspace.numel() * workspace.element_size(),
            rows, cols, row_stride, col_stride, partial, eps, dtype_code(x.dtype), _stream(x),
        ),
        "tb200_rms_norm_bwd",
    )


REDUCE_KINDS = {"sum": 0, "mean": 1, "var": 2, "var_mean": 3}


def reduce_fwd(out_a, out_b, x, y_size, x_size, y_stride, x_stride, kind, correction=0.0):
    _require_cuda(out_a, out_b, x)
    _check(
        load().tb200_reduce_fwd(
            _ptr(out_a), _ptr(out_b), _ptr(x), y_size, x_size, y_stride, x_stride,
            REDUCE_KINDS[kind], float(correction), dtype_code(x.dtype), _stream(x),
        ),
        "tb200_reduce_fwd",
    )


def reduce_bwd(dx, dout_a, dout_b, x, y_size, x_size, y_stride, x_stride, kind, correction=0.0):
    _require_cuda(dx, dout_a, dout_b, x)
    _check(
        load().tb200_reduce_bwd(
            _ptr(dx), _ptr(dout_a), _ptr(dout_b), _ptr(x), y_size, x_size, y_stride, x_stride,
            REDUCE_KINDS[kind], float(correction), dtype_code(dx.dtype), _stream(dx),
        ),
        "tb200_reduce_bwd",
    )


def softmax_fwd(y, x, mask, rows, cols, row_stride, col_stride, mask_row_stride=0,
                mask_col_stride=0):
    _require_cuda(y, x, mask)
    _check(
        load().tb200_softmax_fwd(
            _ptr(y), _ptr(x), _ptr(mask), rows, cols, row_stride, col_stride,
            mask_row_stride, mask_col_stride, dtype_code(x.dtype), _stream(x),
        ),
        "tb200_softmax_fwd",
    )


def softmax_bwd(dx, dy, y, rows, cols, row_stride, col_stride):
    _require_cuda(dx, dy, y)
    _check(
        load().tb200_softmax_bwd(
            _ptr(dx), _ptr(dy), _ptr(y), rows, cols, row_stride, col_stride,
            dtype_code(y.dtype), _stream(y),
        ),
        "tb200_softmax_bwd",
    )


# ---------------------------------------------------------------------- linear / geglu
def linear_fwd(y, x, w, bias, allow_tf32):
    _require_cuda(y, x, w, bias)
    B, M, K = x.shape
    N = w.shape[0]
    _check(
        load().tb200_linear_fwd(
            _ptr(y), _ptr(x), _ptr(w), _ptr(bias), B, M, N, K,
            x.stride(0), x.stride(1), x.stride(2), w.stride(0), w.stride(1),
            int(bool(allow_tf32)), dtype_code(x.dtype), _stream(x),
        ),
        "tb200_linear_fwd",
    )


def linear_bwd_input(dx, dy, w, allow_tf32):
    _require_cuda(dx, dy, w)
    B, M, K = dx.shape
    N = w.shape[0]
    _check(
        load().tb200_linear_bwd_input(
            _ptr(dx), _ptr(dy), _ptr(w), B, M, N, K,
            dx.stride(0), dx.stride(1), dx.stride(2), w.stride(0), w.stride(1),
            int(bool(allow_tf32)), dtype_code(dy.dtype), _stream(dy),
        ),
        "tb200_linear_bwd_input",
    )


def linear_bwd_weight(dw, dy, x, allow_tf32):
    _require_cuda(dw, dy, x)
    B, M, K = x.shape
    N = dw.shape[0]
    _check(
        load().tb200_linear_bwd_weight(
            _ptr(dw), _ptr(dy), _ptr(x), B, M, N, K,
            x.stride(0), x.stride(1), x.stride(2),
            int(bool(allow_tf32)), dtype_code(dy.dtype), _stream(dy),
        ),
        "tb200_linear_bwd_weight",
    )


def linear_bwd_bias_workspace(rows, N):
    return load().tb200_linear_bwd_bias_workspace(rows, N)


def linear_bwd_bias(dbias, dy, workspace, rows, N):
    _require_cuda(dbias, dy, workspace)
    _check(
        load().tb200_linear_bwd_bias(
            _ptr(dbias), _ptr(dy), _ptr(workspace),
            workspace.numel() * workspace.element_size(), rows, N,
            dtype_code(dy.dtype), _stream(dy),
        ),
        "tb200_linear_bwd_bias",
    )


def geglu_fwd(out, state_gate, x, w, bias, gelu_tanh, allow_tf32):
    _require_cuda(out, state_gate, x, w, bias)
    B, M, K = x.shape
    N = w.shape[0]
    _check(
        load().tb200_geglu_fwd(
            _ptr(out), _ptr(state_gate), _ptr(x), _ptr(w), _ptr(bias), B, M, N, K,
            x.stride(0), x.stride(1), x.stride(2), w.stride(0), w.stride(1),
            int(bool(gelu_tanh)), int(bool(allow_tf32)), dtype_code(x.dtype), _stream(x),
        ),
        "tb200_geglu_fwd",
    )


def geglu_fwd_row_scaled(out, state_gate, x, w, bias, row_scale, gelu_tanh):
    """state_gate = row_scale[m] * (x w^T) + bias and out = state * gelu(gate). Returns False when
    the library does not take the inputs on its tensor-core path (the caller then composes
    rms_norm and geglu); raises on any other error."""
    _require_cuda(out, state_gate, x, w, bias, row_scale)
    B, M, K = x.shape
    N = w.shape[0]
    status = load().tb200_geglu_fwd_row_scaled(
        _ptr(out), _ptr(state_gate), _ptr(x), _ptr(w), _ptr(bias), _ptr(row_scale), B, M, N, K,
        x.stride(0), x.stride(1), x.stride(2), w.stride(0), w.stride(1),
        int(bool(gelu_tanh)), dtype_code(x.dtype), _stream(x),
    )
    if status == -2:  # TB200_ERR_UNSUPPORTED
        return False
    _check(status, "tb200_geglu_fwd_row_scaled")
    return True


def geglu_bwd_elementwise(d_state_gate, dout, state_gate, rows, N, gelu_tanh):
    _require_cuda(d_state_gate, dout, state_gate)
    _check(
        load().tb200_geglu_bwd_elementwise(
            _ptr(d_state_gate), _ptr(dout), _ptr(state_gate), rows, N,
            int(bool(gelu_tanh)), dtype_code(dout.dtype), _stream(dout),
        ),
        "tb200_geglu_bwd_elementwise",
    )


def geglu_bwd_elementwise_bias(d_state_gate, dbias, dout, state_gate, workspace, rows, N, gelu_tanh):
    """d_state_gate as geglu_bwd_elementwise, and dbias[N] = its column sums, in one pass."""
    _require_cuda(d_state_gate, dbias, dout, state_gate, workspace)
    _check(
        load().tb200_geglu_bwd_elementwise_bias(
            _ptr(d_state_gate), _ptr(dbias), _ptr(dout), _ptr(state_gate), _ptr(workspace),
            workspace.numel() * workspace.element_size(), rows, N,
            int(bool(gelu_tanh)), dtype_code(dout.dtype), _stream(dout),
        ),
        "tb200_geglu_bwd_elementwise_bias",
    )


# -------------------------------------------------------------------------- attention
def _mask_strides(mask, shape):
    """Element strides of `mask` broadcast to `shape` ([B,H,S,S]); 0 on broadcast dims."""
    view = mask.expand(shape)
    return (c_i64 * 4)(*view.stride())


def attention_fwd(out, lse, q, k, v, mask, is_causal, scale):
    _require_cuda(out, q, k, v, mask)
    B, H, S, D = q.shape
    ms = _mask_strides(mask, (B, H, S, S)) if mask is not None else None
    _check(
        load().tb200_attention_fwd(
            _ptr(out), _ptr(lse), _ptr(q), _ptr(k), _ptr(v), _ptr(mask), B, H, S, D,
            _strides4(q), _strides4(k), _strides4(v), _strides4(out), ms,
            int(bool(is_causal)), scale, dtype_code(q.dtype), _stream(q),
        ),
        "tb200_attention_fwd",
    )


def attention_bwd_workspace(B, H, S, D, dtype):
    return load().tb200_attention_bwd_workspace(B, H, S, D, dtype_code(dtype))


def attention_bwd(dq, dk, dv, dmask, dout, q, k, v, out, lse, mask, workspace, is_causal, scale):
    _require_cuda(dq, dk, dv, dout, q, k, v, out, mask)
    B, H, S, D = q.shape
    ms = _mask_strides(mask, (B, H, S, S)) if mask is not None else None
    _check(
        load().tb200_attention_bwd(
            _ptr(dq), _ptr(dk), _ptr(dv), _ptr(dmask), _ptr(dout), _ptr(q), _ptr(k), _ptr(v),
            _ptr(out), _ptr(lse), _ptr(mask), _ptr(workspace),
            workspace.numel() * workspace.element_size(), B, H, S, D,
            _strides4(q), _strides4(k), _strides4(v), _strides4(out), ms,
            int(bool(is_causal)), scale, dtype_code(q.dtype), _stream(q),
        ),
        "tb200_attention_bwd",
    )
