"""trident_b200: the kernel layer of kakaobrain/trident rebuilt as hand-written sm_100a
CUDA behind a C ABI (libtb200.so), with the reference's function / module API on top.

    import trident_b200 as trident
    y = trident.function.layer_norm(x, (1024,), w, b)
    attn = trident.function.scaled_dot_product_attention(q, k, v, is_causal=True)
"""

from . import config, function, operation, util  # noqa: F401
from .config import *  # noqa: F401,F403
from .module import *  # noqa: F401,F403

__version__ = "0.1.0"
