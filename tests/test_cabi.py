"""The C-ABI library: it loads, exports every symbol the header declares, the ctypes
prototypes cover the same set, and argument validation rejects bad calls before any
launch (so these run without a GPU)."""

import ctypes
import os
import re

import pytest

from trident_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "tb200.h")


def declared_symbols():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(tb200_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_are_exported():
    lib = ctypes.CDLL(_lib.LIB_PATH)
    names = declared_symbols()
    assert len(names) >= 24
    for name in names:
        assert hasattr(lib, name), f"{name} is declared in tb200.h but not exported"


def test_ctypes_prototypes_match_header():
    assert sorted(_lib.SIGNATURES) == declared_symbols()


def test_version_and_error_text():
    lib = _lib.load()
    assert lib.tb200_version() >= 100
    assert isinstance(_lib.last_error(), str)


def test_header_cites_reference_for_every_kernel_entry():
    text = open(HEADER).read()
    for op in ("layer_norm", "rms_norm", "softmax", "linear", "geglu", "attention"):
        assert re.search(rf"trident/kernel/{op}\.py:\d+", text), op
        assert re.search(rf"trident/operation/{op}\.py:\d+", text), op


@pytest.mark.parametrize(
    "call",
    [
        lambda l: l.tb200_layer_norm_fwd(None, None, None, None, None, None, 4, 4, 1e-5, 0, None),
        lambda l: l.tb200_layer_norm_fwd(8, 8, 8, 8, None, None, 4, 0, 1e-5, 0, None),
        lambda l: l.tb200_rms_norm_fwd(8, 8, 8, 8, None, 4, 8, 8, 1, 9, 1e-6, 0, None),
        lambda l: l.tb200_softmax_fwd(None, None, None, 1, 1, 1, 1, 0, 0, 0, None),
        lambda l: l.tb200_softmax_bwd(8, 8, None, 1, 1, 1, 1, 0, None),
        lambda l: l.tb200_linear_fwd(None, None, None, None, 1, 1, 1, 1, 1, 1, 1, 1, 1, 0, 0, None),
        lambda l: l.tb200_geglu_fwd(8, 8, 8, 8, None, 1, 4, 7, 4, 16, 4, 1, 4, 1, 0, 0, 0, None),
        lambda l: l.tb200_geglu_bwd_elementwise(8, 8, 8, 4, 7, 0, 0, None),
        lambda l: l.tb200_geglu_bwd_elementwise_bias(8, 8, 8, 8, 8, 0, 4, 8, 0, 0, None),
        lambda l: l.tb200_attention_fwd(None, None, None, None, None, None, 1, 1, 8, 16, None, None, None, None, None, 0, 1.0, 0, None),
    ],
)
def test_rejected_before_launch(call):
    lib = _lib.load()
    status = call(lib)
    assert status < 0
    assert _lib.last_error() != ""


def test_attention_rejects_bad_head_size_and_mask_plus_causal():
    lib = _lib.load()
    s = (ctypes.c_int64 * 4)(1, 1, 1, 1)
    assert lib.tb200_attention_fwd(8, 8, 8, 8, 8, None, 1, 1, 8, 24, s, s, s, s, None, 0, 1.0, 0, None) == -2
    assert "head size" in _lib.last_error()
    assert lib.tb200_attention_fwd(8, 8, 8, 8, 8, 8, 1, 1, 8, 16, s, s, s, s, s, 1, 1.0, 0, None) == -1
    assert "exclusive" in _lib.last_error()


def test_unknown_dtype_is_rejected():
    lib = _lib.load()
    assert lib.tb200_softmax_bwd(16, 16, 16, 1, 8, 8, 1, 7, None) == -1


def test_workspace_queries():
    lib = _lib.load()
    assert lib.tb200_layer_norm_bwd_workspace(4096, 1024) >= 148 * 2 * 1024 * 4
    assert lib.tb200_rms_norm_bwd_workspace(8192, 4096) >= 148 * 2 * 4096 * 4
    assert lib.tb200_linear_bwd_bias_workspace(8192, 22016) >= 22016 * 4
    assert lib.tb200_linear_bwd_bias_workspace(0, 16) == 0
    # two fp32 row arrays [B,H,S] plus, for 16-bit inputs, an fp32 dq accumulator [B,H,S,D]
    assert lib.tb200_attention_bwd_workspace(2, 3, 128, 64, 0) == 2 * 2 * 3 * 128 * 4
    assert lib.tb200_attention_bwd_workspace(2, 3, 128, 64, 2) == 2 * 2 * 3 * 128 * 4 + 2 * 3 * 128 * 64 * 4
