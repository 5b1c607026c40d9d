from .lightning_attn2 import (  # noqa: F401
    LightningAttention2,
    LightningAttention2NoDecay,
    lightning_attn2,
    lightning_attn2_no_decay,
    lightning_attn2_parallel,
    la_generic,
    la_dkdv,
    lightning_attn_prefill,
    lightning_attn_decode,
)
from .srmsnorm import SimpleRMSNorm, _SrmsNorm, srmsnorm_sigmoid_gate  # noqa: F401
