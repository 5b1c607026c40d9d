"""Quadratic-cost masked-matmul form of decayed causal linear attention in plain torch.

Same function names and numerics as lightning_attn/ops/torch/linear_attention.py: the scores are
computed in the input dtype, multiplied by an fp32 decay mask, rounded back to the input dtype and
multiplied by v. Used as a readable comparison on any device; it is not on the CUDA hot path.
"""
import torch


def get_mask(n, slope=1.0):
    """(n, n) fp32 matrix exp(-slope * (i - j)) for j <= i and 0 above the diagonal
    (lightning_attn/ops/torch/linear_attention.py:4-12)."""
    idx = torch.arange(n, dtype=torch.float32)
    diff = idx[:, None] - idx[None, :]
    expo = torch.where(diff >= 0, -float(slope) * diff, torch.full_like(diff, float("-inf")))
    return torch.exp(expo)


def get_full_mask(n, slopes):
    """(h, n, n) decay masks, or the (n, n) lower-triangular ones matrix when slopes is None
    (lightning_attn/ops/torch/linear_attention.py:15-24)."""
    if slopes is None:
        return torch.tril(torch.ones((n, n)))
    return torch.stack([get_mask(n, float(s)) for s in slopes.reshape(-1)], dim=0)


def linear_attn(q, k, v, s=None):
    """o = ((q k^T) * mask) v (lightning_attn/ops/torch/linear_attention.py:27-34)."""
    n = q.shape[2]
    mask = get_full_mask(n, s).to(q.device).to(torch.float32)
    qk = torch.matmul(q, k.transpose(2, 3))
    qk = (qk.to(torch.float32) * mask).to(q.dtype)
    return torch.matmul(qk, v)
