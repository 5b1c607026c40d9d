"""Generates the golden fixtures in this folder by running the REFERENCE implementation.

Needs the reference checkout (OpenNLPLab/lightning-attention) importable; pass its path as the first
argument or set LIGHTNING_ATTN_REF. Only the reference's torch path is used (`linear_attn` with
autograd, `SimpleRMSNormTorch` with autograd, `_build_slope_tensor`), on CPU, so no GPU is needed:

    python tests/golden/make_golden.py /path/to/lightning-attention

Inputs are stored next to the outputs, so the fixtures do not depend on torch's RNG stream.
"""
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def attn_case(linear_attn, b, h, n, d, e, slopes, dtype, scale, do_mode, seed):
    torch.manual_seed(seed)
    q = (torch.randn((b, h, n, d)) * scale).to(dtype).requires_grad_()
    k = (torch.randn((b, h, n, d)) * scale).to(dtype).requires_grad_()
    v = (torch.randn((b, h, n, e)) * scale).to(dtype).requires_grad_()
    do = torch.ones((b, h, n, e), dtype=dtype) if do_mode == "ones" else (torch.randn((b, h, n, e)) * scale).to(dtype)
    s = None if slopes is None else slopes.to(torch.float32)
    o = linear_attn(q, k, v, s)
    o.backward(do)
    f = lambda t: t.detach().to(torch.float32).numpy()
    out = dict(q=f(q), k=f(k), v=f(v), do=f(do), o=f(o), dq=f(q.grad), dk=f(k.grad), dv=f(v.grad))
    if s is not None:
        out["s"] = s.reshape(-1).numpy()
    return out


def main():
    ref = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("LIGHTNING_ATTN_REF")
    if not ref:
        raise SystemExit("usage: make_golden.py /path/to/lightning-attention")
    sys.path.insert(0, ref)
    from lightning_attn.ops.torch.linear_attention import linear_attn
    from lightning_attn.ops.torch.srmsnorm import SimpleRMSNormTorch
    from lightning_attn.utils import _build_slope_tensor

    torch.set_num_threads(max(1, os.cpu_count() or 1))

    def geometric(h):
        return torch.tensor([2.0 ** (-8.0 * (i + 1) / h) for i in range(h)], dtype=torch.float32).reshape(h, 1, 1)

    cases = {
        # the reference's CPU-runnable configuration: b1 h4 n256 d=e=64 fp32, loss = o.sum()
        "attn_c1_fp32_sum": attn_case(linear_attn, 1, 4, 256, 64, 64, geometric(4), torch.float32, 1.0, "ones", 2024),
        # ragged length, non-power-of-two head count (slopes from _build_slope_tensor), random upstream gradient
        "attn_ragged_fp32": attn_case(linear_attn, 2, 3, 77, 32, 16, _build_slope_tensor(3), torch.float32, 1.0, "randn", 2024),
        # no decay (s=None)
        "attn_nodecay_fp32": attn_case(linear_attn, 1, 2, 130, 16, 32, None, torch.float32, 1.0, "randn", 2024),
        # the reference's own low-precision comparison path (its tests run linear_attn in bf16 on randn/10 inputs)
        "attn_bf16_div10": attn_case(linear_attn, 1, 2, 128, 32, 32, _build_slope_tensor(2), torch.bfloat16, 0.1, "randn", 2024),
    }
    for name, arrs in cases.items():
        np.savez(os.path.join(HERE, name + ".npz"), **arrs)

    # SimpleRMSNorm, fp32 and bf16
    for tag, dtype in (("fp32", torch.float32), ("bf16", torch.bfloat16)):
        torch.manual_seed(2024)
        x = torch.randn((2, 5, 768)).to(dtype).requires_grad_()
        dy = torch.randn((2, 5, 768)).to(dtype)
        y = SimpleRMSNormTorch(768)(x)
        y.backward(dy)
        f = lambda t: t.detach().to(torch.float32).numpy()
        np.savez(os.path.join(HERE, f"srmsnorm_{tag}.npz"), x=f(x), dy=f(dy), y=f(y), dx=f(x.grad), eps=np.float32(1e-6))

    heads = list(range(1, 21)) + [24, 32, 40, 48, 64]
    np.savez(os.path.join(HERE, "slopes.npz"), **{f"h{h}": _build_slope_tensor(h).reshape(-1).numpy() for h in heads})
    print("wrote", sorted(os.listdir(HERE)))


if __name__ == "__main__":
    main()
