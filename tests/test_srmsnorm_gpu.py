"""GPU parity tests of SimpleRMSNorm through the C ABI, with the reference's shapes and tolerance
(tests/ops/test_srmsnorm.py)."""
import os

import numpy as np
import pytest
import torch
from torch.testing import assert_close

import lightning_attention_b200 as la
from oracle import lightning_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda"
ATOL, RTOL = 5e-2, 1e-2  # tests/ops/test_srmsnorm.py:22-23

REF_SHAPES = [(b, n, d) for b in (1, 2, 4, 8) for n in (127, 128, 256, 257, 1024, 1025) for d in (768, 1024)]


def fwd_bwd(mod, x, dy):
    y = mod(x)
    y.backward(dy)
    dx, x.grad = x.grad.clone(), None
    return y.detach(), dx


@pytest.mark.parametrize("b,n,d", REF_SHAPES)
@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
def test_reference_shape_list(cuda_lib, b, n, d, dtype):
    torch.manual_seed(2024)
    x = torch.randn((b, n, d), dtype=dtype, device=DEV).requires_grad_()
    dy = torch.randn((b, n, d), dtype=dtype, device=DEV)
    y_ref, dx_ref = fwd_bwd(la.SimpleRMSNormTorch(d), x, dy)
    y, dx = fwd_bwd(la.SimpleRMSNorm(d), x, dy)
    assert_close(y, y_ref, atol=ATOL, rtol=RTOL)
    assert_close(dx, dx_ref, atol=ATOL, rtol=RTOL)


@pytest.mark.parametrize("rows,dim", [(4 * 8192, 4096), (2 * 32768, 5120)])
def test_baseline_shapes_bf16(cuda_lib, rows, dim):
    torch.manual_seed(2024)
    x = torch.randn((rows, dim), dtype=torch.bfloat16, device=DEV).requires_grad_()
    dy = torch.randn((rows, dim), dtype=torch.bfloat16, device=DEV)
    y, dx = fwd_bwd(la.SimpleRMSNorm(dim), x, dy)
    # fp32 check on a slice of rows (the full fp32 reference would triple the memory), full-tensor sanity on the rest
    sl = slice(0, 2048)
    xs = x.detach()[sl].float().requires_grad_()
    y_ref, dx_ref = fwd_bwd(la.SimpleRMSNormTorch(dim), xs, dy[sl].float())
    assert_close(y[sl].float(), y_ref, atol=ATOL, rtol=RTOL)
    assert_close(dx[sl].float(), dx_ref, atol=ATOL, rtol=RTOL)
    # every output row has unit mean square up to bf16 rounding; dx is orthogonal to x row-wise
    ms = y.float().pow(2).mean(-1)
    assert float((ms - 1).abs().max()) < 2e-2
    xf, dxf = x.detach().float(), dx.float()
    cos = (dxf * xf).sum(-1).abs() / (dxf.norm(dim=-1) * xf.norm(dim=-1) + 1e-20)
    assert float(cos.max()) < 1e-2


@pytest.mark.parametrize("shape", [(3, 100), (5, 7), (2, 3, 1000), (1, 32768), (4, 24576), (2, 6, 136), (0, 64)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_odd_sizes_against_oracle(cuda_lib, shape, dtype):
    if dtype == torch.float32 and shape[-1] * 4 > 65536:
        pytest.skip("row exceeds the 64 KB limit in fp32 (covered by test_row_limit)")
    torch.manual_seed(5)
    x = torch.randn(shape, dtype=dtype, device=DEV).requires_grad_()
    dy = torch.randn(shape, dtype=dtype, device=DEV)
    y, dx = fwd_bwd(la.SimpleRMSNorm(shape[-1]), x, dy)
    assert y.shape == x.shape and dx.shape == x.shape
    if x.numel() == 0:
        return
    xn, dyn = x.detach().float().cpu().numpy(), dy.float().cpu().numpy()
    y_ref, _ = O.srmsnorm_fwd(xn)
    dx_ref = O.srmsnorm_bwd(xn, dyn)
    tol = dict(atol=ATOL, rtol=RTOL) if dtype == torch.bfloat16 else dict(atol=1e-5, rtol=1e-4)
    np.testing.assert_allclose(y.float().cpu().numpy(), y_ref, **tol)
    np.testing.assert_allclose(dx.float().cpu().numpy(), dx_ref, **tol)


def test_unaligned_view_uses_elementwise_kernels(cuda_lib):
    """A row length that is not a multiple of the vector width takes the element-wise kernels."""
    torch.manual_seed(6)
    x = torch.randn((33, 1001), dtype=torch.bfloat16, device=DEV).requires_grad_()
    dy = torch.randn((33, 1001), dtype=torch.bfloat16, device=DEV)
    y, dx = fwd_bwd(la.SimpleRMSNorm(1001), x, dy)
    y_ref, dx_ref = fwd_bwd(la.SimpleRMSNormTorch(1001), x, dy)
    assert_close(y, y_ref, atol=ATOL, rtol=RTOL)
    assert_close(dx, dx_ref, atol=ATOL, rtol=RTOL)


def test_row_limit(cuda_lib):
    x = torch.randn((2, 40000), dtype=torch.bfloat16, device=DEV)
    with pytest.raises(RuntimeError, match="64KB"):
        la.SimpleRMSNorm(40000)(x)


@pytest.mark.parametrize("tag,dtype", [("fp32", torch.float32), ("bf16", torch.bfloat16)])
def test_against_golden_fixtures(cuda_lib, golden_dir, tag, dtype):
    g = dict(np.load(os.path.join(golden_dir, f"srmsnorm_{tag}.npz")))
    x = torch.from_numpy(g["x"]).to(DEV).to(dtype).requires_grad_()
    dy = torch.from_numpy(g["dy"]).to(DEV).to(dtype)
    y, dx = fwd_bwd(la.SimpleRMSNorm(x.shape[-1], float(g["eps"])), x, dy)
    tol = dict(atol=ATOL, rtol=RTOL) if tag == "bf16" else dict(atol=1e-5, rtol=1e-4)
    np.testing.assert_allclose(y.float().cpu().numpy(), g["y"], **tol)
    np.testing.assert_allclose(dx.float().cpu().numpy(), g["dx"], **tol)


def test_fp16_eps_clamp_and_determinism(cuda_lib):
    x = torch.zeros((4, 256), dtype=torch.float16, device=DEV)
    y = la.SimpleRMSNorm(256, eps=1e-9)(x)  # eps is raised to 1.6e-5 for fp16 (srmsnorm.py:80-81): no inf/nan
    assert torch.isfinite(y).all() and float(y.abs().max()) == 0.0
    x = torch.randn((64, 4096), dtype=torch.bfloat16, device=DEV)
    assert torch.equal(la.SimpleRMSNorm(4096)(x), la.SimpleRMSNorm(4096)(x))


@pytest.mark.parametrize("shape", [(4, 1024, 1024), (2, 257, 768), (8192, 4096), (3, 16384), (5, 64), (2, 100), (3, 24576)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
def test_norm_with_sigmoid_gate(cuda_lib, shape, dtype):
    """SimpleRMSNorm(x) * sigmoid(gate), fused forward and backward, against the same expression in fp32 torch with
    autograd; (2, 100) and (3, 24576) take the composed path (rows not vectorisable / too long for the fused kernel)."""
    torch.manual_seed(2025)
    x, g = (torch.randn(shape, dtype=dtype, device=DEV).requires_grad_() for _ in range(2))
    dy = torch.randn(shape, dtype=dtype, device=DEV)
    if shape[-1] * x.element_size() > 65536:  # the norm's own row limit (srmsnorm.py:94-97) applies to the composed path
        with pytest.raises(RuntimeError, match="64KB"):
            la.srmsnorm_sigmoid_gate(x, g)
        return
    y = la.srmsnorm_sigmoid_gate(x, g)
    y.backward(dy)
    xr, gr = (t.detach().float().requires_grad_() for t in (x, g))
    yr = la.SimpleRMSNormTorch(shape[-1])(xr) * torch.sigmoid(gr)
    yr.backward(dy.float())
    assert y.dtype == dtype and y.shape == x.shape
    assert_close(y.float(), yr, atol=ATOL, rtol=RTOL)
    assert_close(x.grad.float(), xr.grad, atol=ATOL, rtol=RTOL)
    assert_close(g.grad.float(), gr.grad, atol=ATOL, rtol=RTOL)


def test_norm_with_sigmoid_gate_against_numpy_oracle(cuda_lib):
    torch.manual_seed(2026)
    x, g, dy = (torch.randn((6, 512), dtype=torch.float32, device=DEV) for _ in range(3))
    x.requires_grad_(); g.requires_grad_()
    y = la.srmsnorm_sigmoid_gate(x, g)
    y.backward(dy)
    f = lambda t: t.detach().cpu().numpy()
    oy, _ = O.srmsnorm_gate_fwd(f(x), f(g))
    dx, dg = O.srmsnorm_gate_bwd(f(x), f(g), f(dy))
    assert O.rel_l2_err(f(y), oy) < 1e-5 and O.rel_l2_err(f(x.grad), dx) < 1e-5 and O.rel_l2_err(f(g.grad), dg) < 1e-5
