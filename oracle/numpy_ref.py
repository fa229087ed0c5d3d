"""Float64 numpy restatement of the hot-path formulas, forward and backward.

Written from the algebra of the reference's Triton kernels (cited per function) with the
oracle's conventions where the two differ (exact erf GELU, exact RMSNorm derivative,
float64 accumulation everywhere). Used on small cases only.
"""

import math

import numpy as np


def _f64(a):
    return None if a is None else np.asarray(a, dtype=np.float64)


# --------------------------------------------------------------------------- LayerNorm
def layer_norm_fwd(x, w, b, eps):
    """trident/kernel/layer_norm.py:72-126: mean, biased variance, rstd, affine."""
    x, w, b = _f64(x), _f64(w), _f64(b)
    mean = x.mean(axis=-1, keepdims=True)
    var = ((x - mean) ** 2).mean(axis=-1, keepdims=True)
    rstd = 1.0 / np.sqrt(var + eps)
    y = (x - mean) * rstd
    if w is not None:
        y = y * w
    if b is not None:
        y = y + b
    return y, mean[..., 0], rstd[..., 0]


def layer_norm_bwd(dy, x, w, eps):
    """trident/kernel/layer_norm.py:188-246 and trident/operation/layer_norm.py:112-122."""
    dy, x, w = _f64(dy), _f64(x), _f64(w)
    n = x.shape[-1]
    _, mean, rstd = layer_norm_fwd(x, None, None, eps)
    xhat = (x - mean[..., None]) * rstd[..., None]
    g = dy if w is None else dy * w
    c1 = (g * xhat).sum(axis=-1, keepdims=True) / n
    c2 = g.sum(axis=-1, keepdims=True) / n
    dx = rstd[..., None] * (g - xhat * c1 - c2)
    dw = (dy * xhat).reshape(-1, n).sum(axis=0)
    db = dy.reshape(-1, n).sum(axis=0)
    return dx, dw, db


# ----------------------------------------------------------------------------- RMSNorm
def rms_partial(n, p):
    return n if p < 0.0 or p > 1.0 else int(n * p)


def rms_norm_fwd(x, p, w, b, eps):
    """trident/kernel/rms_norm.py:74-117 (eps outside the root, leading partial slice)."""
    x, w, b = _f64(x), _f64(w), _f64(b)
    P = rms_partial(x.shape[-1], p)
    rms = np.sqrt((x[..., :P] ** 2).sum(axis=-1, keepdims=True) / P)
    y = x / (rms + eps) * w
    if b is not None:
        y = y + b
    return y, rms[..., 0]


def rms_norm_bwd(dy, x, p, w, eps):
    """Exact derivative of rms_norm_fwd (the reference kernel, trident/kernel/rms_norm.py:213,
    uses rms^2 + eps where the derivative has (rms + eps)^2; they differ at O(eps))."""
    dy, x, w = _f64(dy), _f64(x), _f64(w)
    n = x.shape[-1]
    P = rms_partial(n, p)
    _, rms = rms_norm_fwd(x, p, w, None, eps)
    rms = rms[..., None]
    g = dy * w
    s = (g * x).sum(axis=-1, keepdims=True)
    ind = (np.arange(n) < P).astype(np.float64)
    with np.errstate(divide="ignore", invalid="ignore"):
        second = np.where(rms > 0, ind * x * s / (P * rms * (rms + eps) ** 2), 0.0)
    dx = g / (rms + eps) - second
    dw = (dy * x / (rms + eps)).reshape(-1, n).sum(axis=0)
    db = dy.reshape(-1, n).sum(axis=0)
    return dx, dw, db


# ----------------------------------------------------------------------------- Softmax
def softmax_fwd(x, mask=None, axis=-1):
    """trident/kernel/softmax.py:64-106 and trident/kernel/masked_softmax.py:64-81."""
    x = _f64(x).copy()
    if mask is not None:
        x[np.asarray(mask).astype(bool)] = -np.inf
    m = x.max(axis=axis, keepdims=True)
    e = np.exp(x - m)
    return e / e.sum(axis=axis, keepdims=True)


def softmax_bwd(dy, y, axis=-1):
    """trident/kernel/softmax.py:160-178,223-238: delta = sum(dy*y); dx = y*(dy-delta)."""
    dy, y = _f64(dy), _f64(y)
    delta = (dy * y).sum(axis=axis, keepdims=True)
    return y * (dy - delta)


# ------------------------------------------------------------------------------ Linear
def linear_fwd(x, w, b):
    """trident/language/linear.py:22-95."""
    y = _f64(x) @ _f64(w).T
    return y if b is None else y + _f64(b)


def linear_bwd(dy, x, w):
    """trident/language/linear.py:97-239: input, weight and bias gradients."""
    dy, x, w = _f64(dy), _f64(x), _f64(w)
    dx = dy @ w
    dw = dy.reshape(-1, dy.shape[-1]).T @ x.reshape(-1, x.shape[-1])
    db = dy.reshape(-1, dy.shape[-1]).sum(axis=0)
    return dx, dw, db


# ------------------------------------------------------------------------------- GEGLU
_erf = np.vectorize(math.erf)


def gelu(g, tanh_form=False):
    """trident/language/math/gelu.py:19-24 (tanh form) or the exact erf form."""
    g = _f64(g)
    if tanh_form:
        return 0.5 * g * (1.0 + np.tanh(0.7978845608028654 * g * (1.0 + 0.044715 * g * g)))
    return 0.5 * g * (1.0 + _erf(g / math.sqrt(2.0)))


def gelu_grad(g, tanh_form=False):
    """trident/language/math/gelu.py:26-31 (tanh form) or Phi(g) + g*phi(g)."""
    g = _f64(g)
    if tanh_form:
        a = np.tanh(0.7978845608028654 * g * (1.0 + 0.044715 * g * g))
        return 0.5 * (1.0 + a + g * (1.0 - a * a) * (0.7978845608028654 + 0.1070322244089 * g * g))
    return 0.5 * (1.0 + _erf(g / math.sqrt(2.0))) + g * np.exp(-0.5 * g * g) / math.sqrt(2.0 * math.pi)


def geglu_fwd(x, w, b, tanh_form=False):
    """trident/kernel/geglu.py:124-177: state = first half, gate = second half."""
    sg = linear_fwd(x, w, b)
    X = sg.shape[-1] // 2
    return sg[..., :X] * gelu(sg[..., X:], tanh_form), sg


def geglu_bwd(dout, x, w, b, tanh_form=False):
    """trident/kernel/geglu.py:236-242 followed by the Linear backward on d_state_gate."""
    dout = _f64(dout)
    _, sg = geglu_fwd(x, w, b, tanh_form)
    X = sg.shape[-1] // 2
    state, gate = sg[..., :X], sg[..., X:]
    dsg = np.concatenate([dout * gelu(gate, tanh_form), dout * state * gelu_grad(gate, tanh_form)], axis=-1)
    return linear_bwd(dsg, x, w)


# --------------------------------------------------------------------------- Attention
def attention_fwd(q, k, v, mask=None, causal=False, scale=None):
    """trident/kernel/attention.py:115-165 without tiling: returns (out, lse) with the
    natural-log sum of exponentials per score row."""
    q, k, v = _f64(q), _f64(k), _f64(v)
    S, D = q.shape[-2], q.shape[-1]
    scale = 1.0 / math.sqrt(D) if scale is None else scale
    s = scale * (q @ np.swapaxes(k, -1, -2))
    if mask is not None:
        s = s + _f64(mask)
    if causal:
        s = np.where(np.tril(np.ones((S, S), dtype=bool)), s, -np.inf)
    m = s.max(axis=-1, keepdims=True)
    e = np.exp(s - m)
    l = e.sum(axis=-1, keepdims=True)
    return (e / l) @ v, (m + np.log(l))[..., 0]


def attention_bwd(dout, q, k, v, mask=None, causal=False, scale=None):
    """trident/kernel/attention.py:283-339 without tiling: (dq, dk, dv, dmask)."""
    dout, q, k, v = _f64(dout), _f64(q), _f64(k), _f64(v)
    S, D = q.shape[-2], q.shape[-1]
    scale = 1.0 / math.sqrt(D) if scale is None else scale
    out, lse = attention_fwd(q, k, v, mask, causal, scale)
    s = scale * (q @ np.swapaxes(k, -1, -2))
    if mask is not None:
        s = s + _f64(mask)
    if causal:
        s = np.where(np.tril(np.ones((S, S), dtype=bool)), s, -np.inf)
    p = np.exp(s - lse[..., None])
    delta = (out * dout).sum(axis=-1, keepdims=True)
    dv = np.swapaxes(p, -1, -2) @ dout
    dp = dout @ np.swapaxes(v, -1, -2)
    ds = p * (dp - delta)
    dq = scale * (ds @ k)
    dk = scale * (np.swapaxes(ds, -1, -2) @ q)
    return dq, dk, dv, ds


def var_mean_fwd(x, axis, correction=1):
    """sum, mean and variance along `axis` (trident/language/sum.py, mean.py, var.py: centred
    squares divided by n - correction)."""
    x = _f64(x)
    n = x.shape[axis]
    total = x.sum(axis=axis)
    mean = total / n
    var = ((x - np.expand_dims(mean, axis)) ** 2).sum(axis=axis) / (n - correction)
    return total, mean, var


def var_mean_bwd(dvar, dmean, x, axis, correction=1):
    """dx = dvar * 2 (x - mean) / (n - correction) + dmean / n (trident/kernel/var_mean.py:86-131)."""
    x = _f64(x)
    n = x.shape[axis]
    mean = np.expand_dims(x.mean(axis=axis), axis)
    return (np.expand_dims(_f64(dvar), axis) * 2.0 * (x - mean) / (n - correction)
            + np.expand_dims(_f64(dmean), axis) / n)
