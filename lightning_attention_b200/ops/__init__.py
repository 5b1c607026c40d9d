from .lightning_attn_interface import lightning_attn_func, is_support, next_power_of_2  # noqa: F401
from .torch import linear_attn, SimpleRMSNormTorch  # noqa: F401
from .cuda import (  # noqa: F401
    lightning_attn2,
    lightning_attn2_no_decay,
    lightning_attn2_parallel,
    LightningAttention2,
    LightningAttention2NoDecay,
    SimpleRMSNorm,
    la_generic,
    la_dkdv,
    lightning_attn_prefill,
    lightning_attn_decode,
    srmsnorm_sigmoid_gate,
)

__all__ = [
    "lightning_attn_func", "is_support", "next_power_of_2", "linear_attn", "SimpleRMSNormTorch",
    "lightning_attn2", "lightning_attn2_no_decay", "lightning_attn2_parallel", "LightningAttention2",
    "LightningAttention2NoDecay", "SimpleRMSNorm", "la_generic", "la_dkdv", "lightning_attn_prefill", "lightning_attn_decode", "srmsnorm_sigmoid_gate",
]
