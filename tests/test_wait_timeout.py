"""A bounded wait that runs out: the abort path of the tensor-core kernels, executed once.

Every mbarrier wait of those kernels has a time limit; when one expires the CTA raises an abort
flag, records a code in the device status word, lets its roles run to their end, drains what
they have in flight and frees its tensor memory. The test hook `tb200_test_wait_fault(1)` makes
exactly that happen in the attention forward: the limit shrinks to about a millisecond and the
producer of one CTA leaves out the copy of one key tile (it touches no memory a normal launch
would not touch), so the MMA issuer waits for a tile that never arrives. Nothing faults and
nothing hangs: the launch ends by itself, the status word is non-zero, and the next normal call
on the same context is correct.
"""

import math

import pytest
import torch

import trident_b200 as trident
from oracle import torch_oracle
from tests import util
from trident_b200 import _lib

pytestmark = pytest.mark.gpu


def test_expired_wait_sets_the_status_word_and_the_context_stays_usable(device):
    dt = torch.bfloat16
    B, H, S, D = 1, 2, 256, 64
    q, k, v = (util.randn(B, H, S, D, seed=s, dtype=dt, device=device) for s in (1, 2, 3))
    _lib.device_status(reset=True)
    assert _lib.device_status() == 0
    out = torch.empty_like(q)
    lse = torch.empty(B, H, S, device=device, dtype=torch.float32)
    old = _lib.test_wait_fault(1)
    try:
        _lib.attention_fwd(out, lse, q, k, v, None, False, 1.0 / math.sqrt(D))
        assert _lib.last_kernel() == "attn_tcgen05"
        torch.cuda.synchronize()  # returns: the kernel ended by itself
    finally:
        _lib.test_wait_fault(old)
    code = _lib.device_status(reset=True)
    assert code != 0, "the expired wait was not recorded"
    assert _lib.device_status() == 0
    # the same context, the same kernel, without the hook: correct result and a clean status
    got = trident.function.scaled_dot_product_attention(q, k, v)
    want = torch_oracle.scaled_dot_product_attention(q.float().cpu(), k.float().cpu(), v.float().cpu())
    util.assert_half_close(got, want, dt, atol=1e-2, ulps=1.0, what="forward after the aborted launch")
    assert _lib.device_status() == 0
