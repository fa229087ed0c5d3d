"""Guard regions around every buffer a library call writes.

`guards()` is a context manager that wraps each launch wrapper of `trident_b200._lib`: every
output tensor and workspace of the call is replaced by a view into a larger allocation whose
margins (64 KiB before and after) hold a byte pattern; after the call has completed the margins
are compared with the pattern and the result is copied back into the caller's tensor. A kernel
that stores, reduces or bulk-copies outside the buffer it was given therefore fails the test
that ran it, with the entry point and the argument named. This is the out-of-bounds-write check
of these tests (they compare bytes after the fact; nothing is made to fault).
"""

import contextlib

import torch

from trident_b200 import _lib

GUARD = 64 * 1024
PATTERN = 0xA5

# positions of the tensors each wrapper writes (outputs and workspaces)
WRITTEN = {
    "layer_norm_fwd": (0, 1, 2),
    "layer_norm_bwd": (0, 1, 2, 8),
    "layer_norm_bwd_static": (0, 1, 2),
    "rms_norm_fwd": (0, 1),
    "rms_norm_bwd": (0, 1, 2, 7),
    "reduce_fwd": (0, 1),
    "reduce_bwd": (0,),
    "softmax_fwd": (0,),
    "softmax_bwd": (0,),
    "linear_fwd": (0,),
    "linear_bwd_input": (0,),
    "linear_bwd_weight": (0,),
    "linear_bwd_bias": (0, 2),
    "geglu_fwd": (0, 1),
    "geglu_bwd_elementwise": (0,),
    "geglu_bwd_elementwise_bias": (0, 1, 4),
    "attention_fwd": (0, 1),
    "attention_bwd": (0, 1, 2, 3, 11),
}


class GuardViolation(AssertionError):
    pass


class _Guarded:
    def __init__(self, original):
        self.original = original
        nbytes = original.numel() * original.element_size()
        padded = (nbytes + 255) // 256 * 256
        self.raw = torch.full((GUARD + padded + GUARD,), PATTERN, dtype=torch.uint8, device=original.device)
        self.nbytes, self.padded = nbytes, padded
        middle = self.raw[GUARD:GUARD + nbytes]
        self.view = middle.view(original.dtype).view(original.shape) if nbytes else original

    def check(self, where):
        lo = self.raw[:GUARD]
        hi = self.raw[GUARD + self.nbytes:]
        for name, part in (("before", lo), ("after", hi)):
            bad = (part != PATTERN).nonzero()
            if bad.numel():
                first = int(bad[0])
                offset = first - GUARD if name == "before" else first
                raise GuardViolation(
                    f"{where}: {bad.numel()} guard bytes {name} the buffer were overwritten "
                    f"(first at byte offset {offset:+d} from the buffer's {'start' if name == 'before' else 'end'}; "
                    f"buffer of {self.nbytes} bytes, shape {tuple(self.original.shape)}, {self.original.dtype})"
                )

    def copy_back(self):
        if self.nbytes:
            self.original.copy_(self.view)


def _wrap(name, fn, stats):
    positions = WRITTEN[name]

    def guarded(*args, **kwargs):
        args = list(args)
        swapped = []
        for pos in positions:
            t = args[pos] if pos < len(args) else None
            if t is None or not torch.is_tensor(t) or not t.is_cuda or not t.is_contiguous():
                continue
            g = _Guarded(t)
            args[pos] = g.view
            swapped.append((pos, g))
        result = fn(*args, **kwargs)
        torch.cuda.synchronize()
        for pos, g in swapped:
            g.check(f"{name} argument {pos}")
            g.copy_back()
        stats[name] = stats.get(name, 0) + 1
        return result

    return guarded


@contextlib.contextmanager
def guards():
    """Installs the guarded wrappers; yields a dict counting the guarded calls per entry point."""
    stats = {}
    saved = {name: getattr(_lib, name) for name in WRITTEN}
    try:
        for name, fn in saved.items():
            setattr(_lib, name, _wrap(name, fn, stats))
        yield stats
    finally:
        for name, fn in saved.items():
            setattr(_lib, name, fn)
