"""Package-level switches, same names as trident/config.py:16-17.

`use_autotune` is kept so that code written for the reference keeps importing; the CUDA
kernels choose their launch shapes analytically, so it has no effect. `use_trace` turns
the NVTX ranges of `util.push_trace` / `util.pop_trace` on.
"""

use_autotune = True
use_trace = False

# GELU flavour of GEGLU: False = exact erf form (what the reference's test oracle
# computes, tests/test_geglu.py:22-24), True = the tanh approximation of the reference's
# Triton kernel (trident/language/math/gelu.py:19-31).
geglu_tanh_approximation = False
