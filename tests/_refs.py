"""Test-only helpers: a differentiable fp32 torch restatement of the block recurrence for sizes the
numpy oracle would take too long on (it runs on the GPU next to the kernel under test), and the
tolerances every parity test uses."""
import numpy as np
import torch

# Stated tolerance for bf16 results against an fp32 reference.
REL_L2_TOL = 1e-2
MAX_ABS_TOL = 2e-2  # on the reference tests' randn/10 inputs; N(0,1) inputs use it relative to max|ref|


def geometric_slopes(h, device="cpu"):
    return torch.tensor([2.0 ** (-8.0 * (i + 1) / h) for i in range(h)], dtype=torch.float32, device=device).reshape(h, 1, 1)


def torch_la_reference(q, k, v, s=None, block=256):
    """fp32, differentiable: per block o = (q k^T * M) v + (q kv) * lambda^r ; kv = lambda^B kv + (k * lambda^(B-r))^T v
    (the recurrence of lightning_attn2.py:55-85 with a larger block)."""
    q, k, v = q.float(), k.float(), v.float()
    b, h, n, d = q.shape
    e = v.shape[-1]
    dev = q.device
    sv = torch.zeros(h, device=dev) if s is None else s.float().reshape(-1)[:h].to(dev)
    sv = sv.view(1, h, 1, 1)
    r = torch.arange(block, device=dev, dtype=torch.float32)
    diff = r[:, None] - r[None, :]
    mask = torch.where(diff >= 0, torch.exp(-sv * diff.clamp(min=0)), torch.zeros((), device=dev))
    qdec = torch.exp(-sv * r.view(1, 1, block, 1))
    kdec = torch.exp(-sv * (block - r).view(1, 1, block, 1))
    bdec = torch.exp(-sv * block)
    kv = torch.zeros(b, h, d, e, device=dev)
    outs = []
    for i in range(0, n, block):
        qi, ki, vi = q[:, :, i:i + block], k[:, :, i:i + block], v[:, :, i:i + block]
        m = qi.shape[2]
        o = ((qi @ ki.transpose(2, 3)) * mask[:, :, :m, :m]) @ vi + (qi @ kv) * qdec[:, :, :m]
        outs.append(o)
        if m == block:
            kv = bdec * kv + (ki * kdec).transpose(2, 3) @ vi
    return torch.cat(outs, dim=2)


def errs(x, ref):
    x = x.detach().double()
    ref = ref.detach().double()
    diff = (x - ref)
    max_abs = float(diff.abs().max()) if ref.numel() else 0.0
    den = float(ref.norm())
    rel = float(diff.norm()) / den if den > 0 else float(diff.norm())
    return max_abs, rel, float(ref.abs().max()) if ref.numel() else 0.0


def assert_parity(x, ref, name, scaled_inputs):
    """rel-L2 <= 1e-2 always; max-abs <= 2e-2 absolute for randn/10 inputs, relative to max|ref| otherwise."""
    max_abs, rel, ref_max = errs(x, ref)
    assert np.isfinite(max_abs), f"{name}: non-finite values"
    assert rel <= REL_L2_TOL, f"{name}: rel-L2 {rel:.3e} > {REL_L2_TOL}"
    bound = MAX_ABS_TOL if scaled_inputs else MAX_ABS_TOL * max(ref_max, 1.0)
    assert max_abs <= bound, f"{name}: max-abs {max_abs:.3e} > {bound:.3e} (max|ref| {ref_max:.3e})"
