"""CPU oracle for the trident_b200 kernels. TEST INFRASTRUCTURE ONLY.

Nothing in the product path (the `trident_b200` package, the C-ABI library) imports this
package. It is used by tests/, by the smoke check and by the CPU-baseline / reference arm
of bench.py as the checker and as the timed CPU baseline.

Two layers:
  * torch_oracle — the torch eager callables that the reference's own tests compare its
    kernels against (tests/test_layer_norm.py, test_rms_norm.py, test_softmax.py,
    test_masked_softmax.py, test_linear.py, test_geglu.py, test_attention.py).
  * numpy_ref   — a float64 numpy restatement of the same formulas, forward and backward,
    written from the reference kernels' algebra; it cross-checks torch_oracle on small
    cases and produces the committed golden vectors.

Pinning: PARITY UNPINNED against the reference's own kernels. The reference's tests hold no
golden vectors or known-answer fixtures (their inputs are unseeded random tensors), and its
Triton kernels cannot execute here (no GPU in the build container; on a GPU box `import trident`
fails under the installed Triton release). The oracle is therefore pinned only to the exact torch
callables those tests compare against, cross-checked by the independent float64 restatement
and by the committed seeded vectors under tests/golden/ (generated from the torch oracle by
tests/golden/make_golden.py; tests/golden/README.md lists them).
"""
