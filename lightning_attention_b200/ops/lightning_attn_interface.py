"""User-facing wrapper with the reference's signature (lightning_attn/ops/lightning_attn_interface.py:16-65).

The reference pads e to a power of two and splits d > 128 into 64-wide slices whose partial
outputs it sums, because its Triton kernels need power-of-two tiles. The CUDA kernels take any
d <= 256 and e <= 256 that are multiples of 16, so here padding only happens for sizes that are not
multiples of 16, and splitting only for d > 256 (the product q.k is additive over feature slices) and
e > 256 (output columns are independent).
"""
import math

import torch
import torch.nn.functional as F

from .cuda import lightning_attn2, lightning_attn2_no_decay

_MAX_D = 256  # largest d (and e) the kernels take in one piece


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
        # q.k is additive over feature slices and the output is linear in it: d > 256 runs as slices whose partial outputs are
        # summed in the tensors' dtype (what the reference does from d > 128 on with 64-wide slices,
        # lightning_attn_interface.py:34-55). 128 < d <= 256 stays in one piece: cutting it at 128 so that every piece runs
        # on the warp-specialised kernel was measured on the README shape (b2 h12 n2048 d=e=192) and is 3x slower there
        # (four sub-problems, their launches and the adds and concatenations around them: 1.25 ms against 0.42 ms).
        if d <= _MAX_D:
            return fn(q, k, v1)
        o1 = 0
        for start in range(0, d, _MAX_D):
            o1 = o1 + fn(q[..., start:start + _MAX_D], k[..., start:start + _MAX_D], v1)
        return o1

    # Output columns are independent of each other: e > 256, which the backward kernels do not take in one piece (dq
    # contracts over e), runs as column slices of v whose outputs are concatenated; autograd sums their dq and dk.
    if v.shape[-1] > _MAX_D:
        o = torch.cat([over_d(v[..., start:start + _MAX_D]) for start in range(0, v.shape[-1], _MAX_D)], dim=-1)
    else:
        o = over_d(v)
    return o[..., :e] if o.shape[-1] != e else o
