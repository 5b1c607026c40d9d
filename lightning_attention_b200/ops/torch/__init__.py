from .linear_attention import linear_attn, get_full_mask, get_mask  # noqa: F401
from .srmsnorm import SimpleRMSNormTorch  # noqa: F401
