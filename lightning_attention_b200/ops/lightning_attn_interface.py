"""User-facing wrapper with the reference's signature (lightning_attn/ops/lightning_attn_interface.py:16-65).

The reference pads e to a power of two and splits d > 128 into 64-wide slices whose partial
outputs it sums, because its Triton kernels need power-of-two tiles. The CUDA kernels take any
d <= 256 and e <= 256 that are multiples of 16, so here padding only happens for sizes that are not
multiples of 16. d > 128 is split into slices of at most 128 features (the product q.k is additive over feature slices) so
that every slice runs on the fast kernel, and e > 128 into column slices (output columns are independent) for the same reason.
"""
import math

import torch
import torch.nn.functional as F

from .cuda import lightning_attn2, lightning_attn2_no_decay

_MAX_D = 256   # largest d (and e) the kernels take in one piece
_FAST_D = 128  # largest d of the warp-specialised block kernel; wider d runs a slower serial-phase kernel


def is_support(dim):
    """The reference's quirky support test, kept for API parity (lightning_attn_interface.py:8-9):
    falsy exactly when dim divides 16. It is not used to gate anything here."""
    return 16 % dim


def next_power_of_2(n):
    return 2 ** (int(math.ceil(math.log(n, 2))))


def _pad_last(x, mult):
    r = (-x.shape[-1]) % mult
    return F.pad(x, (0, r)) if r else x


def lightning_attn_func(q, k, v, s=None, variant="chunk_loop"):
    """o_t = sum_{j<=t} exp(-s (t-j)) (q_t . k_j) v_j per head; s=None means no decay.

    `variant` is accepted for compatibility ("chunk_loop" or "parallel"); one implementation serves both.
    """
    if variant not in ("chunk_loop", "parallel"):
        raise ValueError(f"unknown variant {variant!r}")
    e = v.shape[-1]
    q = _pad_last(q, 16)
    k = _pad_last(k, 16)
    v = _pad_last(v, 16)
    d = q.shape[-1]

    def fn(q1, k1, v1):
        return lightning_attn2_no_decay(q1, k1, v1) if s is None else lightning_attn2(q1, k1, v1, s)

    def over_d(v1):
        # q.k is additive over feature slices and the output is linear in it, so d > 128 runs as slices of at most 128
        # features on the fast kernel and the partial outputs are summed in the tensors' dtype - what the reference does with
        # 64-wide slices (lightning_attn_interface.py:34-55). One piece up to d = 256 is also possible (lightning_attn2
        # called directly takes it) but runs the serial-phase kernel, which is slower.
        if d <= _FAST_D:
            return fn(q, k, v1)
        o1 = 0
        for start in range(0, d, _FAST_D):
            o1 = o1 + fn(q[..., start:start + _FAST_D], k[..., start:start + _FAST_D], v1)
        return o1

    # Output columns are independent of each other, so wide e runs as column slices of v whose outputs are concatenated
    # (autograd sums their dq, dk): at most 128 columns each, because the backward pass contracts over e (dq) and only
    # takes the fast kernels, fused dk+dv sweep included, up to 128; beyond 256 the backward kernels do not take e at all.
    if v.shape[-1] > _FAST_D:
        o = torch.cat([over_d(v[..., start:start + _FAST_D]) for start in range(0, v.shape[-1], _FAST_D)], dim=-1)
    else:
        o = over_d(v)
    return o[..., :e] if o.shape[-1] != e else o
