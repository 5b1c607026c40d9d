"""SimpleRMSNorm (no weight) as a torch.autograd.Function backed by liblightning_b200.so.

Mirrors lightning_attn/ops/triton/srmsnorm.py:76-185: same class names, same fp16 eps clamp, same
64 KB-per-row limit and error, (x, rstd) saved for backward.
"""
import torch

from ... import _lib


class _SrmsNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, eps):
        _lib.require_cuda(x)
        if x.dtype == torch.float16:
            eps = max(eps, 1.6e-5)  # srmsnorm.py:80-81
        N = x.shape[-1]
        if N * x.element_size() > 65536:
            raise RuntimeError("This layer norm doesn't support feature dim >= 64KB.")  # srmsnorm.py:96-97
        x_arg = x.reshape(-1, N)
        if not x_arg.is_contiguous():
            x_arg = x_arg.contiguous()
        M = x_arg.shape[0]
        y = torch.empty_like(x_arg)
        rstd = torch.empty((M,), dtype=torch.float32, device=x.device)
        with torch.cuda.device(x.device):
            rc = _lib.lib().lab200_srmsnorm_fwd(x_arg.data_ptr(), y.data_ptr(), rstd.data_ptr(), M, N, float(eps),
                                                _lib.dtype_code(x.dtype), _lib.stream_ptr(x.device))
        _lib.check(rc, "lab200_srmsnorm_fwd")
        ctx.save_for_backward(x_arg, rstd)
        return y.reshape(x.shape)

    @staticmethod
    def backward(ctx, dy):
        x, rstd = ctx.saved_tensors
        M, N = x.shape
        dy_arg = dy.reshape(-1, N).contiguous()
        assert dy_arg.numel() == x.numel(), "gradient and input sizes differ"  # srmsnorm.py:155-157
        if dy_arg.dtype != x.dtype:
            dy_arg = dy_arg.to(x.dtype)
        dx = torch.empty_like(dy_arg)
        with torch.cuda.device(x.device):
            rc = _lib.lib().lab200_srmsnorm_bwd(x.data_ptr(), dy_arg.data_ptr(), rstd.data_ptr(), dx.data_ptr(), M, N,
                                                _lib.dtype_code(x.dtype), _lib.stream_ptr(x.device))
        _lib.check(rc, "lab200_srmsnorm_bwd")
        return dx.reshape(dy.shape), None


class SimpleRMSNorm(torch.nn.Module):
    """y = x / sqrt(mean(x^2, -1) + eps), no learnable weight (srmsnorm.py:178-185)."""

    def __init__(self, dim: int, eps: float = 1e-6):
        super().__init__()
        self.eps = eps
        self.dim = dim

    def forward(self, x):
        return _SrmsNorm.apply(x, self.eps)
