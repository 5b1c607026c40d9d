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


class _SrmsNormGate(torch.autograd.Function):
    """y = SimpleRMSNorm(x) * sigmoid(gate) in one kernel each way (the norm + gate epilogue of the reference's example
    caller, examples/module/tnl_attn.py:66-69, with SimpleRMSNorm as the norm)."""

    @staticmethod
    def forward(ctx, x, gate, eps):
        _lib.require_cuda(x, gate)
        if gate.shape != x.shape or gate.dtype != x.dtype:
            raise RuntimeError(f"gate must match x in shape and dtype; got {tuple(gate.shape)} {gate.dtype} vs {tuple(x.shape)} {x.dtype}")
        if x.dtype == torch.float16:
            eps = max(eps, 1.6e-5)
        N = x.shape[-1]
        x_arg = _aligned16(x.reshape(-1, N).contiguous())
        g_arg = _aligned16(gate.reshape(-1, N).contiguous())
        M = x_arg.shape[0]
        y = torch.empty_like(x_arg)
        rstd = torch.empty((M,), dtype=torch.float32, device=x.device)
        with torch.cuda.device(x.device):
            rc = _lib.lib().lab200_srmsnorm_gate_fwd(x_arg.data_ptr(), g_arg.data_ptr(), y.data_ptr(), rstd.data_ptr(), M, N,
                                                     float(eps), _lib.dtype_code(x.dtype), _lib.stream_ptr(x.device))
        _lib.check(rc, "lab200_srmsnorm_gate_fwd")
        ctx.save_for_backward(x_arg, g_arg, rstd)
        return y.reshape(x.shape)

    @staticmethod
    def backward(ctx, dy):
        x, g, rstd = ctx.saved_tensors
        M, N = x.shape
        dy_arg = dy.reshape(-1, N).contiguous()
        if dy_arg.dtype != x.dtype:
            dy_arg = dy_arg.to(x.dtype)
        dy_arg = _aligned16(dy_arg)
        dx = torch.empty_like(x)
        dg = torch.empty_like(x)
        with torch.cuda.device(x.device):
            rc = _lib.lib().lab200_srmsnorm_gate_bwd(x.data_ptr(), g.data_ptr(), dy_arg.data_ptr(), rstd.data_ptr(),
                                                     dx.data_ptr(), dg.data_ptr(), M, N, _lib.dtype_code(x.dtype),
                                                     _lib.stream_ptr(x.device))
        _lib.check(rc, "lab200_srmsnorm_gate_bwd")
        return dx.reshape(dy.shape), dg.reshape(dy.shape), None


def _aligned16(t):
    """The fused kernels use 128-bit loads: a contiguous view whose storage offset is not 16-byte aligned (a slice of a flat
    buffer) is copied once; fresh allocations are always aligned."""
    return t if t.data_ptr() % 16 == 0 else t.clone()


def _gate_rows_supported(x):
    epv = 4 if x.dtype == torch.float32 else 8
    N = x.shape[-1]
    return N % epv == 0 and N // epv <= 2048


def srmsnorm_sigmoid_gate(x, gate, eps=1e-6):
    """SimpleRMSNorm(x) * sigmoid(gate). One fused kernel forward and one backward for rows of up to 16384 16-bit (8192
    fp32) elements that are a multiple of the 128-bit vector width; other rows compose SimpleRMSNorm with torch ops."""
    if _gate_rows_supported(x):
        return _SrmsNormGate.apply(x, gate, eps)
    return _SrmsNorm.apply(x, eps) * torch.sigmoid(gate)


class SimpleRMSNorm(torch.nn.Module):
    """y = x / sqrt(mean(x^2, -1) + eps), no learnable weight (srmsnorm.py:178-185)."""

    def __init__(self, dim: int, eps: float = 1e-6):
        super().__init__()
        self.eps = eps
        self.dim = dim

    def forward(self, x):
        return _SrmsNorm.apply(x, self.eps)
