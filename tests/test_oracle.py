"""CPU tests: the numpy oracle against the fixtures generated from the reference, and its internal
consistency (naive form == block recurrences == generic product; known-answer cases)."""
import os

import numpy as np
import pytest

from oracle import lightning_oracle as O


def load(golden_dir, name):
    return dict(np.load(os.path.join(golden_dir, name + ".npz")))


@pytest.mark.parametrize("name", ["attn_c1_fp32_sum", "attn_ragged_fp32", "attn_nodecay_fp32"])
def test_naive_matches_reference_fp32(golden_dir, name):
    g = load(golden_dir, name)
    s = g.get("s")
    o = O.linear_attn(g["q"], g["k"], g["v"], s)
    dq, dk, dv = O.linear_attn_bwd(g["q"], g["k"], g["v"], s, g["do"])
    # the reference ran in fp32; the oracle in fp64 => agreement to fp32 rounding of O(n)-term sums
    for got, key in ((o, "o"), (dq, "dq"), (dk, "dk"), (dv, "dv")):
        assert O.rel_l2_err(got, g[key]) < 2e-6, key
        assert O.max_abs_err(got, g[key]) < 1e-3 * max(1.0, float(np.abs(g[key]).max())), key


@pytest.mark.parametrize("name", ["attn_c1_fp32_sum", "attn_ragged_fp32", "attn_nodecay_fp32"])
@pytest.mark.parametrize("block", [64, 128])
def test_blockwise_matches_reference_fp32(golden_dir, name, block):
    g = load(golden_dir, name)
    s = g.get("s")
    o = O.la2_fwd_blockwise(g["q"], g["k"], g["v"], s, block=block)
    dq, dk, dv = O.la2_bwd_blockwise(g["q"], g["k"], g["v"], s, g["do"], block=block)
    for got, key in ((o, "o"), (dq, "dq"), (dk, "dk"), (dv, "dv")):
        assert O.rel_l2_err(got, g[key]) < 2e-6, key


def test_reference_bf16_path_within_stated_tolerance(golden_dir):
    """The reference's own low-precision path (what its tests compare against) stays within the stated
    bf16 tolerance of the fp64 oracle on randn/10 inputs: the tolerance is attainable."""
    g = load(golden_dir, "attn_bf16_div10")
    o = O.linear_attn(g["q"], g["k"], g["v"], g["s"])
    dq, dk, dv = O.linear_attn_bwd(g["q"], g["k"], g["v"], g["s"], g["do"])
    for got, key in ((o, "o"), (dq, "dq"), (dk, "dk"), (dv, "dv")):
        assert O.rel_l2_err(g[key], got) < 1e-2, key
        assert O.max_abs_err(g[key], got) < 2e-2, key


def test_generic_product_roles(golden_dir):
    """forward / dq / dk / dv are the four role assignments of the generic product."""
    g = load(golden_dir, "attn_ragged_fp32")
    q, k, v, do, s = g["q"], g["k"], g["v"], g["do"], g["s"]
    o, _ = O.la_generic(q, k, v, s)
    dq, _ = O.la_generic(do, v, k, s)
    dk, _ = O.la_generic(v, do, q, s, reverse=True)
    dv, _ = O.la_generic(k, q, do, s, reverse=True)
    for got, key in ((o, "o"), (dq, "dq"), (dk, "dk"), (dv, "dv")):
        assert O.rel_l2_err(got, g[key]) < 2e-6, key


def test_slopes_match_reference(golden_dir):
    g = load(golden_dir, "slopes")
    for key, ref in g.items():
        h = int(key[1:])
        assert np.array_equal(O.build_slopes(h), ref), key


@pytest.mark.parametrize("tag", ["fp32", "bf16"])
def test_srmsnorm_matches_reference(golden_dir, tag):
    g = load(golden_dir, "srmsnorm_" + tag)
    y, _ = O.srmsnorm_fwd(g["x"], float(g["eps"]))
    dx = O.srmsnorm_bwd(g["x"], g["dy"], float(g["eps"]))
    # tolerance of the reference's own test (tests/ops/test_srmsnorm.py:22-23); fp32 is far tighter
    atol, rtol = (5e-2, 1e-2) if tag == "bf16" else (1e-5, 1e-5)
    np.testing.assert_allclose(y, g["y"], atol=atol, rtol=rtol)
    np.testing.assert_allclose(dx, g["dx"], atol=atol, rtol=rtol)


def test_known_answer_counting():
    """s = 0, q = k = 1/sqrt(d), v = 1  =>  o_t = t + 1."""
    b, h, n, d, e = 1, 2, 200, 16, 8
    q = np.full((b, h, n, d), 1 / np.sqrt(d))
    v = np.ones((b, h, n, e))
    o = O.la2_fwd_blockwise(q, q, v, None)
    np.testing.assert_allclose(o[0, 0, :, 0], np.arange(1, n + 1), rtol=1e-12)


def test_known_answer_geometric():
    """q = k = e_1, v = e_1 with decay  =>  o_t = (1 - lambda^(t+1)) / (1 - lambda)."""
    n, d = 150, 16
    q = np.zeros((1, 1, n, d)); q[..., 0] = 1
    s = np.array([0.25])
    o = O.la2_fwd_blockwise(q, q, q, s)
    lam = np.exp(-0.25)
    np.testing.assert_allclose(o[0, 0, :, 0], (1 - lam ** (np.arange(n) + 1)) / (1 - lam), rtol=1e-12)


def test_block_size_invariance():
    rng = np.random.default_rng(1)
    q, k, v = (rng.standard_normal((1, 3, 300, x)) for x in (16, 16, 32))
    s = O.build_slopes(3)
    o64 = O.la2_fwd_blockwise(q, k, v, s, block=64)
    o128 = O.la2_fwd_blockwise(q, k, v, s, block=128)
    assert O.max_abs_err(o64, o128) < 1e-10


def test_d_split_identity():
    """Summing outputs over feature slices of q, k equals the unsplit result (the reference's d > 128 path,
    lightning_attn_interface.py:34-55)."""
    rng = np.random.default_rng(2)
    q, k, v = (rng.standard_normal((1, 2, 100, x)) for x in (192, 192, 24))
    s = O.build_slopes(2)
    full = O.linear_attn(q, k, v, s)
    parts = sum(O.linear_attn(q[..., i:i + 64], k[..., i:i + 64], v, s) for i in range(0, 192, 64))
    assert O.max_abs_err(full, parts) < 1e-9


@pytest.mark.parametrize("reverse", [False, True])
@pytest.mark.parametrize("scale", [1.0, 1e-3, 0.0])
def test_sequence_parallel_chain_equals_single(reverse, scale):
    """Sharding the sequence over R ranks and chaining the decayed states reproduces the unsharded result."""
    rng = np.random.default_rng(3)
    b, h, R, L, dk, dv = 1, 3, 4, 128, 16, 32
    n = R * L
    a, bm, c = (rng.standard_normal((b, h, n, x)) for x in (dk, dk, dv))
    s = O.build_slopes(h) * scale if scale > 0 else None
    full, full_state = O.la_generic(a, bm, c, s, reverse=reverse)
    sl = [slice(r * L, (r + 1) * L) for r in range(R)]
    local = [O.la_generic(a[:, :, x], bm[:, :, x], c[:, :, x], s, reverse=reverse)[1] for x in sl]
    incoming = O.sp_incoming_states(local, s, L, reverse=reverse)
    outs = [O.la_generic(a[:, :, x], bm[:, :, x], c[:, :, x], s, reverse=reverse, state_in=incoming[r])[0]
            for r, x in enumerate(sl)]
    assert O.max_abs_err(np.concatenate(outs, axis=2), full) < 1e-9


def test_state_and_decode_chain_matches_definition():
    """The exported state (entering token n, ragged n included) and the decode step, against the O(n^2) definition."""
    rng = np.random.default_rng(5)
    b, h, n, d, e = 1, 3, 300, 16, 24
    q, k = rng.standard_normal((2, b, h, n, d))
    v = rng.standard_normal((b, h, n, e))
    s = O.build_slopes(h) * 0.3
    ref = O.linear_attn(q, k, v, s)
    n1, n2 = 171, 290
    o1, st = O.la_generic(q[:, :, :n1], k[:, :, :n1], v[:, :, :n1], s)
    assert O.max_abs_err(st, O.state_entering(k[:, :, :n1], v[:, :, :n1], s)) < 1e-10
    o2, st = O.la_generic(q[:, :, n1:n2], k[:, :, n1:n2], v[:, :, n1:n2], s, state_in=st)
    assert O.max_abs_err(st, O.state_entering(k[:, :, :n2], v[:, :, :n2], s)) < 1e-10
    outs = [o1, o2]
    for t in range(n2, n):
        o, st = O.decode_step(q[:, :, t], k[:, :, t], v[:, :, t], s, st)
        outs.append(o[:, :, None])
    assert O.max_abs_err(np.concatenate(outs, axis=2), ref) < 1e-10


def test_gated_norm_gradients_match_autograd():
    """oracle.srmsnorm_gate_* against torch autograd of SimpleRMSNorm(x) * sigmoid(g) in fp64 on the CPU."""
    import torch

    rng = np.random.default_rng(6)
    x, g, dy = rng.standard_normal((3, 5, 64))
    xt, gt = (torch.tensor(t, dtype=torch.float64, requires_grad=True) for t in (x, g))
    y = xt * torch.rsqrt(xt.pow(2).mean(-1, keepdim=True) + 1e-6) * torch.sigmoid(gt)
    y.backward(torch.tensor(dy))
    oy, _ = O.srmsnorm_gate_fwd(x, g)
    dx, dg = O.srmsnorm_gate_bwd(x, g, dy)
    assert O.max_abs_err(oy, y.detach().numpy()) < 1e-12
    assert O.max_abs_err(dx, xt.grad.numpy()) < 1e-12
    assert O.max_abs_err(dg, gt.grad.numpy()) < 1e-12
