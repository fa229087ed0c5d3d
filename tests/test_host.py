"""Host-side logic that needs no GPU: shape plumbing, argument errors raised before any
kernel call, module construction, workload sharding."""

import pytest
import torch

import trident_b200 as trident
import workloads
from trident_b200 import _lib, util
from trident_b200.operation.masked_softmax import as_byte_mask
from trident_b200.operation.rms_norm import partial_size


def test_is_pow2():
    assert [util.is_pow2(v) for v in (0, 1, 2, 3, 4, 6, 1024)] == [False, True, True, False, True, False, True]


def test_size_and_stride():
    x = torch.empty(3, 5)
    assert util.size_and_stride(x, 1) == (3, 5, 5, 1)
    assert util.size_and_stride(x, -1) == (3, 5, 5, 1)
    assert util.size_and_stride(x, None) == (3, 5, 5, 1)
    assert util.size_and_stride(x, 0) == (5, 3, 1, 5)
    with pytest.raises(ValueError):
        util.size_and_stride(torch.empty(2, 3, 4), 0)


def test_partial_size():
    assert partial_size(10, 0.5) == 5
    assert partial_size(1000, 1.0) == 1000
    assert partial_size(16, -1.0) == 16
    assert partial_size(16, 1.5) == 16


def test_as_byte_mask():
    like = torch.empty(2, 4)
    m = torch.tensor([[0, 1, 0, 2], [1, 0, 0, 0]])
    assert as_byte_mask(m, like).dtype == torch.uint8
    assert as_byte_mask(m, like).tolist() == [[0, 1, 0, 1], [1, 0, 0, 0]]
    assert as_byte_mask(m.bool(), like).tolist() == [[0, 1, 0, 1], [1, 0, 0, 0]]
    assert as_byte_mask(m.float(), like).tolist() == [[0, 1, 0, 1], [1, 0, 0, 0]]


def test_modules_and_reprs():
    ln = trident.LayerNorm(8)
    assert ln.weight.shape == (8,) and torch.all(ln.weight == 1) and torch.all(ln.bias == 0)
    assert repr(ln).endswith("backend=Trident)")
    assert trident.LayerNorm((4, 8), elementwise_affine=False).weight is None
    rms = trident.RMSNorm(8, bias=True)
    assert torch.all(rms.weight == 1) and torch.all(rms.bias == 0) and rms.p == -1.0 and rms.eps == 1e-5
    lin = trident.Linear(16, 8)
    assert lin.weight.shape == (8, 16) and lin.bias.shape == (8,)
    assert set(lin.state_dict()) == {"weight", "bias"}
    gg = trident.GEGLU(16, 8, bias=False)
    assert gg.bias is None and gg.weight.abs().max() <= 0.25
    assert "dim=1, backend=Trident" in repr(trident.Softmax(1))
    assert "dim=None, backend=Trident" in repr(trident.MaskedSoftmax())
    assert "dim=0, backend=Trident" in repr(trident.Sum(0)) and "dim=1, backend=Trident" in repr(trident.Mean(1))
    assert "dim=1, correction=0, backend=Trident" in repr(trident.Var(1, 0))
    assert "dim=None, correction=1, backend=Trident" in repr(trident.VarMean())
    assert trident.use_trace is False and trident.use_autotune is True


def test_attention_argument_errors_before_any_launch():
    f = trident.function.scaled_dot_product_attention
    q = torch.randn(1, 1, 8, 16)
    with pytest.raises(ValueError, match="dimension"):
        f(q[0], q[0], q[0])
    with pytest.raises(ValueError, match="power of 2"):
        f(q[..., :6], q[..., :6], q[..., :6])  # head size
    with pytest.raises(ValueError, match="both attn_mask and is_causal"):
        f(q, q, q, attn_mask=torch.zeros(1, 1, 8, 8), is_causal=True)
    with pytest.raises(ValueError, match="dropout"):
        f(q, q, q, dropout_p=1.0)
    with pytest.raises(ValueError, match="same shape"):
        f(q, q[:, :, :4], q)


def test_no_cpu_fallback():
    """CPU tensors are refused: the product path has no fallback implementation."""
    x = torch.randn(4, 8)
    with pytest.raises(_lib.Tb200Error, match="CUDA tensors only"):
        trident.function.softmax(x, 1)
    with pytest.raises(_lib.Tb200Error, match="CUDA tensors only"):
        trident.function.layer_norm(x, (8,))
    with pytest.raises(_lib.Tb200Error, match="CUDA tensors only"):
        trident.function.var_mean(x, 1)
    with pytest.raises(_lib.Tb200Error, match="CUDA tensors only"):
        trident.function.sum(x, 0)


def test_dtype_code():
    assert _lib.dtype_code(torch.float32) == 0 and _lib.dtype_code(torch.bfloat16) == 2
    with pytest.raises(ValueError):
        _lib.dtype_code(torch.int64)


@pytest.mark.parametrize("name", list(workloads.WORKLOADS))
def test_shards_concatenate_to_the_single_rank_problem(name):
    wl = workloads.WORKLOADS[name]
    kw = {"scale": 32}
    if name.startswith("attention"):
        kw = {"scale": 16, "S": 64}
    if name == "geglu":
        kw["n_scale"] = 64
    whole = wl.make(0, 1, "cpu", **kw)
    for world in (2, 4, 8):
        parts = [wl.make(r, world, "cpu", **kw) for r in range(world)]
        for key in ("x", "q", "k", "v", "dy", "mask"):
            if key in whole:
                flat = (lambda v: v.flatten(0, -3)) if whole[key].dim() > 2 else (lambda v: v)
                cat = torch.cat([flat(p[key]) for p in parts])
                assert torch.equal(cat, flat(whole[key])), (name, key, world)
        for key in ("w", "b"):
            if key in whole:
                assert all(torch.equal(p[key], whole[key]) for p in parts)
    with pytest.raises(ValueError):
        workloads.owned_blocks(0, 3)


def test_workload_work_figures_at_full_size():
    """Algorithmic bytes / flops of the full configurations (no tensors are allocated)."""

    class Meta:
        def __init__(self, shape, esize):
            self.shape, self._n, self._e = shape, 1, esize
            for s in shape:
                self._n *= s

        def numel(self):
            return self._n

        def element_size(self):
            return self._e

    W = workloads.WORKLOADS
    assert W["layer_norm"].work({"x": Meta((4096, 1024), 4)}) == 83886080
    assert W["softmax"].work({"x": Meta((16384, 4096), 2)}) == 671088640
    assert W["masked_softmax"].work({"x": Meta((16384, 4096), 2), "mask": Meta((16384, 4096), 1)}) == 738197504
    assert W["rms_norm"].work({"x": Meta((8192, 4096), 2)}) == 335544320
    assert W["geglu"].work({"x": Meta((8192, 4096), 2), "w": Meta((22016, 4096), 2)}) == 4432406249472
    assert W["attention_causal"].work({"q": Meta((4, 32, 4096, 128), 2)}) == 1924145348608
    assert W["attention_masked"].work({"q": Meta((8, 16, 16384, 64), 2)}) == 30786325577728
