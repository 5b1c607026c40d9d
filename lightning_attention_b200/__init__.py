"""Lightning Attention-2 and SimpleRMSNorm for NVIDIA B200 (sm_100a).

Same operator surface as OpenNLPLab/lightning-attention (``lightning_attn/__init__.py:1-2``):
``lightning_attn_func``, ``lightning_attn2``, ``lightning_attn2_no_decay``, ``SimpleRMSNorm``,
``linear_attn``, ``SimpleRMSNormTorch``, ``_build_slope_tensor``, ``get_memory``; the device code is
hand-written CUDA behind the C ABI of ``liblightning_b200.so``.
"""
from .ops import *  # noqa: F401,F403
from .utils import *  # noqa: F401,F403
from .utils import _build_slope_tensor  # noqa: F401  (underscore names are not star-exported)

__version__ = "0.1.0"
