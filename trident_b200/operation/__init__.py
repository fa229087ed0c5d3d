from .attention import Attention
from .geglu import GEGLU
from .layer_norm import LayerNorm
from .linear import Linear
from .masked_softmax import MaskedSoftmax
from .reduce import Mean, Sum, Var, VarMean
from .rms_norm import RMSNorm
from .rms_norm_geglu import RMSNormGEGLU
from .softmax import Softmax

__all__ = [
    "Attention", "GEGLU", "LayerNorm", "Linear", "MaskedSoftmax", "Mean", "RMSNorm", "RMSNormGEGLU", "Softmax", "Sum", "Var", "VarMean",
]
