"""CPU tests of the host side: the C-ABI library loads and exports what include/*.h declares, argument
validation, planning helpers, and the Python mirror of the reference's interface. No kernel runs here."""
import ctypes
import os
import re

import numpy as np
import pytest
import torch

import lightning_attention_b200 as la
from lightning_attention_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    names = set()
    inc = os.path.join(ROOT, "include")
    for fn in os.listdir(inc):
        if fn.endswith(".h"):
            text = open(os.path.join(inc, fn)).read()
            text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
            names |= set(re.findall(r"\b(lab200_\w+)\s*\(", text))
    return sorted(names)


def test_library_exports_every_declared_symbol():
    L = _lib.lib()
    names = declared_symbols()
    assert len(names) >= 10
    for n in names:
        assert hasattr(L, n), f"{n} declared in include/ but not exported"
    assert sorted(_lib.EXPORTS) == [n for n in names if n in _lib.EXPORTS]
    assert set(_lib.EXPORTS) <= set(names)


def test_version_and_error_strings():
    L = _lib.lib()
    assert L.lab200_version() >= 100
    assert L.lab200_error_string(0) == b"ok"
    for code in (1, 2, 3, 4, 5, 6, 101, 102, 103):
        assert len(L.lab200_error_string(code)) > 3
    assert L.lab200_error_string(9999) == b"unknown error"


def test_attention_argument_validation_needs_no_gpu():
    L = _lib.lib()
    buf = (ctypes.c_char * 4096)()
    p = ctypes.addressof(buf)
    p = (p + 15) & ~15
    ws = 1024
    # dk not a multiple of 16, dk too large, bad dtype, missing pointers, misaligned pointer
    assert L.lab200_la_generic(p, p, p, None, p, None, None, p, ws, 1, 1, 128, 24, 64, 0, 0, 0, _lib.BF16, None) == 1
    assert L.lab200_la_generic(p, p, p, None, p, None, None, p, ws, 1, 1, 128, 272, 64, 0, 0, 0, _lib.BF16, None) == 1
    assert L.lab200_la_generic(p, p, p, None, p, None, None, p, ws, 1, 1, 128, 64, 64, 0, 0, 0, _lib.F32, None) == 2
    assert L.lab200_la_generic(None, p, p, None, p, None, None, p, ws, 1, 1, 128, 64, 64, 0, 0, 0, _lib.BF16, None) == 1
    assert L.lab200_la_generic(p + 2, p, p, None, p, None, None, p, ws, 1, 1, 128, 64, 64, 0, 0, 0, _lib.BF16, None) == 6
    assert L.lab200_la_generic(p, p, p, None, p, None, None, p, ws, 0, 1, 128, 64, 64, 0, 0, 0, _lib.BF16, None) == 1
    assert L.lab200_la2_fwd(p, p, p, None, p, p, ws, 1, 1, 0, 64, 64, 0, _lib.BF16, None) == 1
    # a reverse-time sweep cannot take an incoming state when the sequence ends in a ragged block
    assert L.lab200_la_generic(p, p, p, None, p, p, None, p, ws, 1, 1, 200, 64, 64, 1, 0, 0, _lib.BF16, None) == 1
    # the projection-layout flag needs whole batches of heads and dk <= 128
    assert L.lab200_la_generic(p, p, p, None, p, None, None, p, ws, 3, 2, 128, 64, 64, 0, 0, 0, _lib.BF16 | 0x100, None) == 1
    assert L.lab200_la_generic(p, p, p, None, p, None, None, p, ws, 2, 2, 128, 192, 64, 0, 0, 0, _lib.BF16 | 0x100, None) == 1
    assert L.lab200_la2_bwd(p, p, p, None, p, p, p, p, p, ws, 1, 1, 128, 64, 20, 0, _lib.BF16, None) == 1


def test_srmsnorm_argument_validation_needs_no_gpu():
    L = _lib.lib()
    buf = (ctypes.c_char * 256)()
    p = ctypes.addressof(buf)
    assert L.lab200_srmsnorm_fwd(p, p, p, 4, 40000, 1e-6, _lib.BF16, None) == 1  # row > 64 KB
    assert L.lab200_srmsnorm_fwd(p, p, p, 4, 128, 1e-6, 7, None) == 2
    assert L.lab200_srmsnorm_fwd(p, p, p, 0, 128, 1e-6, _lib.BF16, None) == 0  # empty input: nothing to do
    assert L.lab200_srmsnorm_bwd(p, None, p, p, 4, 128, _lib.BF16, None) == 1


def test_workspace_and_chunk_planning():
    L = _lib.lib()
    assert L.lab200_la_workspace_bytes(128, 32768, 128, 128, 1) == 256
    assert L.lab200_la_workspace_bytes(16, 32768, 128, 128, 8) == 256 + 16 * 8 * 128 * 128 * 4
    # never more chunks than 128-token blocks
    assert L.lab200_la_workspace_bytes(1, 256, 64, 64, 100) == 256 + 2 * 64 * 64 * 4
    # plenty of (batch, head) pairs: one serial sweep each; few pairs: split the sequence
    assert L.lab200_la_plan_chunks(128, 32768, 128, 128) == 1
    assert L.lab200_la_plan_chunks(16, 32768, 128, 128) > 1
    assert L.lab200_la_plan_chunks(1, 128, 128, 128) == 1


def test_ops_refuse_cpu_tensors():
    q = torch.randn(1, 2, 128, 64, dtype=torch.bfloat16)
    with pytest.raises(RuntimeError, match="CUDA"):
        la.lightning_attn_func(q, q, q, la._build_slope_tensor(2))
    with pytest.raises(RuntimeError, match="CUDA"):
        la.SimpleRMSNorm(64)(q)


def test_public_names_match_reference_surface():
    for name in ("lightning_attn_func", "lightning_attn2", "lightning_attn2_no_decay", "lightning_attn2_parallel",
                 "linear_attn", "SimpleRMSNorm", "SimpleRMSNormTorch", "_build_slope_tensor", "get_memory",
                 "is_support", "next_power_of_2"):
        assert hasattr(la, name) or hasattr(la.ops, name), name
    assert la.next_power_of_2(192) == 256 and la.next_power_of_2(64) == 64
    assert la.is_support(16) == 0 and la.is_support(128) == 16  # the reference's quirk, lightning_attn_interface.py:8-9
    with pytest.raises(ValueError):
        la.lightning_attn_func(None, None, torch.zeros(1, 1, 1, 16), None, variant="nope")


def test_slope_tensor_matches_reference(golden_dir):
    g = np.load(os.path.join(golden_dir, "slopes.npz"))
    for key in g.files:
        h = int(key[1:])
        t = la._build_slope_tensor(h)
        assert t.shape == (h, 1, 1) and t.dtype == torch.float32
        assert np.array_equal(t.reshape(-1).numpy(), g[key]), key


@pytest.mark.parametrize("name", ["attn_c1_fp32_sum", "attn_ragged_fp32", "attn_nodecay_fp32"])
def test_torch_naive_path_matches_reference(golden_dir, name):
    """The package's plain-torch `linear_attn` (same name as the reference's) reproduces the reference on CPU."""
    g = dict(np.load(os.path.join(golden_dir, name + ".npz")))
    q, k, v, do = (torch.from_numpy(g[x]).requires_grad_() for x in ("q", "k", "v", "do"))
    s = torch.from_numpy(g["s"]).reshape(-1, 1, 1) if "s" in g else None
    o = la.linear_attn(q, k, v, s)
    o.backward(do.detach())
    for got, key in ((o, "o"), (q.grad, "dq"), (k.grad, "dk"), (v.grad, "dv")):
        np.testing.assert_allclose(got.detach().numpy(), g[key], rtol=2e-4, atol=2e-4 * float(np.abs(g[key]).max()))


def test_torch_srmsnorm_matches_reference(golden_dir):
    g = dict(np.load(os.path.join(golden_dir, "srmsnorm_fp32.npz")))
    x = torch.from_numpy(g["x"]).requires_grad_()
    y = la.SimpleRMSNormTorch(768)(x)
    y.backward(torch.from_numpy(g["dy"]))
    np.testing.assert_allclose(y.detach().numpy(), g["y"], rtol=1e-5, atol=1e-6)
    np.testing.assert_allclose(x.grad.numpy(), g["dx"], rtol=1e-4, atol=1e-6)


@pytest.mark.parametrize("name", ["attn_c1_fp32_sum", "attn_ragged_fp32", "attn_nodecay_fp32"])
@pytest.mark.parametrize("block", [64, 256])
def test_gpu_side_torch_reference_is_pinned_to_the_reference(golden_dir, name, block):
    """tests/_refs.py:torch_la_reference - the fp32 torch block recurrence most GPU parity tests compare with - reproduces
    the reference's outputs and autograd gradients on the golden fixtures (ragged n and non-power-of-two head counts
    included) and agrees with the numpy oracle; run here on the CPU, it is the same code the GPU tests run on the device."""
    import sys

    sys.path.insert(0, os.path.join(ROOT, "tests"))
    from _refs import torch_la_reference
    from oracle import lightning_oracle as O

    g = dict(np.load(os.path.join(golden_dir, name + ".npz")))
    q, k, v, do = (torch.from_numpy(g[x]).requires_grad_() for x in ("q", "k", "v", "do"))
    s = torch.from_numpy(g["s"]).reshape(-1, 1, 1) if "s" in g else None
    o = torch_la_reference(q, k, v, s, block=block)
    o.backward(do.detach())
    odq, odk, odv = O.linear_attn_bwd(g["q"], g["k"], g["v"], g.get("s"), g["do"])
    oo = O.linear_attn(g["q"], g["k"], g["v"], g.get("s"))
    for got, key, orc in ((o, "o", oo), (q.grad, "dq", odq), (k.grad, "dk", odk), (v.grad, "dv", odv)):
        got = got.detach().numpy()
        assert O.rel_l2_err(got, g[key]) < 5e-6, (key, "vs the reference fixture")
        assert O.rel_l2_err(got, orc) < 5e-6, (key, "vs the numpy oracle")


def test_backward_workspace_covers_every_product_of_the_backward_pass():
    """lab200_la2_bwd runs products with (dk, dv) = (e, d) and (d, e); each plans its own chunks, and the size the Python
    layer asks for must cover the largest (d != e with few (batch, head) pairs used to come out too small)."""
    L = _lib.lib()
    for (b, h, n, d, e) in ((1, 32, 2048, 128, 256), (1, 32, 4096, 128, 192), (1, 48, 2048, 192, 64), (1, 40, 2048, 64, 192),
                            (4, 32, 32768, 128, 128), (1, 4, 131072, 128, 128)):
        need = L.lab200_la2_bwd_workspace_bytes(b, h, n, d, e, 0)
        assert need >= L.lab200_la_workspace_bytes(b * h, n, e, d, 0)
        assert need >= L.lab200_la_workspace_bytes(b * h, n, d, e, 0)
        assert need >= 256


def test_status_queries_need_no_gpu():
    L = _lib.lib()
    assert L.lab200_last_status() == 0  # no device, no ring: nothing to report
