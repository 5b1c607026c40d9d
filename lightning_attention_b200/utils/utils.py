"""Helpers with the reference's names (lightning_attn/utils/utils.py)."""
import math

import torch


def _slopes(h: int):
    """ALiBi-style decay rates. Power-of-two head counts get the geometric sequence
    2^(-8(i+1)/h); other counts take the sequence of the next lower power of two and fill up with
    every second entry of the sequence for twice that power (lightning_attn/utils/utils.py:6-24)."""
    if h < 1:
        raise ValueError("need at least one head")
    p = 2 ** int(math.floor(math.log2(h)))
    if p == h:
        start = 2 ** (-(2 ** -(math.log2(h) - 3)))
        return [start * start**i for i in range(h)]
    return _slopes(p) + _slopes(2 * p)[0::2][: h - p]


def _build_slope_tensor(n_attention_heads: int):
    """Per-head decay rates as an fp32 tensor of shape (h, 1, 1) (lightning_attn/utils/utils.py:6-31)."""
    return torch.tensor(_slopes(n_attention_heads), dtype=torch.float32).reshape(n_attention_heads, 1, 1)


def get_memory(device):
    """Peak allocated MiB on `device` since the last call (lightning_attn/utils/utils.py:34-38)."""
    mb_used = torch.cuda.max_memory_allocated(device) / 1024 / 1024
    torch.cuda.reset_peak_memory_stats(device)
    return mb_used
