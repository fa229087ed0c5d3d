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

Pinning: the reference's tests hold no golden vectors or known-answer fixtures (their
inputs are unseeded random tensors), and its Triton kernels cannot execute in the build
container (no GPU; incompatible Triton release). The oracle is therefore pinned to the
exact torch callables those tests name, cross-checked by the independent float64
restatement, and, where the reference's Triton source could be executed under Triton's
CPU interpreter, to vectors generated from it (tests/golden/README.md says which).
"""
