"""Plain-torch SimpleRMSNorm with the reference's name (lightning_attn/ops/torch/srmsnorm.py:9-20)."""
import torch
import torch.nn as nn


class SimpleRMSNormTorch(nn.Module):
    def __init__(self, dim: int, eps: float = 1e-6):
        super().__init__()
        self.eps = eps

    def forward(self, x):
        xf = x.float()
        return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + self.eps)).type_as(x)
