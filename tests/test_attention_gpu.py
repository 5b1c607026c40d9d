"""GPU parity tests of the attention path. Everything goes through the C ABI (ctypes), either directly or
via the autograd Functions. References: the numpy oracle (small sizes), the golden fixtures generated
from the reference, and an fp32 torch restatement of the block recurrence (large sizes)."""
import os

import numpy as np
import pytest
import torch

import lightning_attention_b200 as la
from lightning_attention_b200 import _lib
from lightning_attention_b200.ops.cuda.lightning_attn2 import la_generic
from oracle import lightning_oracle as O

from _refs import assert_parity, errs, geometric_slopes, torch_la_reference

pytestmark = pytest.mark.gpu
DEV = "cuda"

# the reference's own shape list, tests/ops/test_lightning2.py:9-28
REF_SHAPES = [
    (6, 8, 256, 128, 64), (6, 8, 512, 128, 64), (6, 8, 1024, 128, 64), (6, 8, 2048, 128, 64),
    (6, 8, 4096, 128, 64), (6, 8, 8192, 128, 64), (6, 8, 2048, 32, 64), (6, 8, 2048, 64, 64),
    (6, 12, 2048, 128, 64), (6, 16, 2048, 128, 64), (6, 20, 2048, 128, 64), (1, 8, 2048, 128, 64),
    (2, 8, 2048, 128, 64), (3, 8, 2048, 128, 64), (6, 8, 913, 128, 64), (6, 8, 513, 128, 64),
    (6, 8, 1213, 128, 64), (6, 8, 2048, 16, 64),
]


def make_inputs(b, h, n, d, e, dtype, scale, seed=2024):
    torch.manual_seed(seed)
    q = (torch.randn((b, h, n, d), device=DEV) * scale).to(dtype).requires_grad_()
    k = (torch.randn((b, h, n, d), device=DEV) * scale).to(dtype).requires_grad_()
    v = (torch.randn((b, h, n, e), device=DEV) * scale).to(dtype).requires_grad_()
    do = (torch.randn((b, h, n, e), device=DEV) * scale).to(dtype)
    return q, k, v, do


def run_fwd_bwd(fn, q, k, v, do):
    o = fn(q, k, v)
    o.backward(do)
    grads = (q.grad, k.grad, v.grad)
    q.grad = k.grad = v.grad = None
    return (o.detach(),) + tuple(g.detach() for g in grads)


def compare_with_torch_reference(q, k, v, do, s, got, scaled, tag):
    qr, kr, vr = (t.detach().float().requires_grad_() for t in (q, k, v))
    ref = run_fwd_bwd(lambda a, b_, c: torch_la_reference(a, b_, c, s), qr, kr, vr, do.float())
    for x, r, name in zip(got, ref, ("o", "dq", "dk", "dv")):
        assert_parity(x, r, f"{tag}:{name}", scaled)


@pytest.mark.parametrize("b,h,n,d,e", REF_SHAPES)
def test_reference_shape_list_bf16(cuda_lib, b, h, n, d, e):
    """Same shapes, seed, randn/10 inputs and slopes as tests/ops/test_lightning2.py:33-58, with real assertions."""
    q, k, v, do = make_inputs(b, h, n, d, e, torch.bfloat16, 0.1)
    s = la._build_slope_tensor(h).to(DEV)
    got = run_fwd_bwd(lambda a, b_, c: la.lightning_attn2(a, b_, c, s), q, k, v, do)
    compare_with_torch_reference(q, k, v, do, s, got, True, f"decay{(b, h, n, d, e)}")


@pytest.mark.parametrize("b,h,n,d,e", REF_SHAPES)
def test_reference_shape_list_fp16(cuda_lib, b, h, n, d, e):
    """The reference's second dtype (tests/ops/test_lightning2.py:35), all 18 shapes. fp16 rounds finer than
    bf16, so the same tolerance applies with room to spare; the running state is carried in fp32 and only its
    tensor-core copy is fp16, which randn/10 inputs keep far from the fp16 range limit."""
    q, k, v, do = make_inputs(b, h, n, d, e, torch.float16, 0.1)
    s = la._build_slope_tensor(h).to(DEV)
    got = run_fwd_bwd(lambda a, b_, c: la.lightning_attn2(a, b_, c, s), q, k, v, do)
    compare_with_torch_reference(q, k, v, do, s, got, True, f"fp16{(b, h, n, d, e)}")


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("b,h,n,d,e", REF_SHAPES)
def test_reference_shape_list_no_decay(cuda_lib, b, h, n, d, e, dtype):
    """tests/ops/test_lightning2_no_decay.py:8-56 (s=None): all 18 shapes, both dtypes."""
    q, k, v, do = make_inputs(b, h, n, d, e, dtype, 0.1)
    got = run_fwd_bwd(lambda a, b_, c: la.lightning_attn2_no_decay(a, b_, c), q, k, v, do)
    compare_with_torch_reference(q, k, v, do, None, got, True, f"nodecay{(b, h, n, d, e)}")


@pytest.mark.parametrize("slopes", ["formula", "build"])
def test_readme_example_config(cuda_lib, slopes):
    """b2 h12 n2048 d=e=192 bf16, N(0,1) inputs, loss = o.sum(), through lightning_attn_func
    (examples/ops/example_lightning_attn.py)."""
    b, h, n, d, e = 2, 12, 2048, 192, 192
    q, k, v, _ = make_inputs(b, h, n, d, e, torch.bfloat16, 1.0)
    s = (geometric_slopes(h, DEV) if slopes == "formula" else la._build_slope_tensor(h).to(DEV))
    do = torch.ones((b, h, n, e), device=DEV, dtype=torch.bfloat16)
    got = run_fwd_bwd(lambda a, b_, c: la.lightning_attn_func(a, b_, c, s), q, k, v, do)
    compare_with_torch_reference(q, k, v, do, s, got, False, f"readme-{slopes}")


@pytest.mark.parametrize("n", [512, 2048, 8192])
@pytest.mark.parametrize("decay", [True, False])
def test_benchmark_config_small_n(cuda_lib, n, decay):
    """b4 h32 d=e=128 bf16 N(0,1) (benchmarks/benchmark_lightning2.py:99-102), with and without decay."""
    b, h, d = 4, 32, 128
    q, k, v, do = make_inputs(b, h, n, d, d, torch.bfloat16, 1.0)
    s = la._build_slope_tensor(h).to(DEV) if decay else None
    fn = (lambda a, b_, c: la.lightning_attn_func(a, b_, c, s))
    got = run_fwd_bwd(fn, q, k, v, do)
    compare_with_torch_reference(q, k, v, do, s, got, False, f"bench-n{n}-decay{decay}")


def test_benchmark_config_full_size_sampled(cuda_lib):
    """b4 h32 n32768 d=e=128: the whole tensor is computed; three (batch, head) pairs are checked against the
    fp32 recurrence, and the result must be linear in v (a size-independent property)."""
    b, h, n, d = 4, 32, 32768, 128
    q, k, v, do = make_inputs(b, h, n, d, d, torch.bfloat16, 1.0)
    s = la._build_slope_tensor(h).to(DEV)
    o, dq, dk, dv = run_fwd_bwd(lambda a, b_, c: la.lightning_attn2(a, b_, c, s), q, k, v, do)
    for (ib, ih) in ((0, 0), (1, 17), (3, 31)):
        sl = (slice(ib, ib + 1), slice(ih, ih + 1))
        qs, ks, vs, dos = (t[sl].detach() for t in (q, k, v, do))
        qr, kr, vr = (t.float().requires_grad_() for t in (qs, ks, vs))
        ref = run_fwd_bwd(lambda a, b_, c: torch_la_reference(a, b_, c, s[ih:ih + 1]), qr, kr, vr, dos.float())
        for x, r, name in zip((o, dq, dk, dv), ref, ("o", "dq", "dk", "dv")):
            assert_parity(x[sl], r, f"full-size({ib},{ih}):{name}", False)
    with torch.no_grad():
        o2 = la.lightning_attn2(q, k, (2 * v.detach()).to(torch.bfloat16), s)  # exact doubling in bf16
    assert torch.equal(o2.float(), 2 * o.float())


def c_generic(cuda_lib, a, bm, c, s, reverse, state_in, want_state, chunks, state_only=False):
    """Direct ctypes call of lab200_la_generic with raw pointers (no Python op layer in between)."""
    b, h, n, dk = bm.shape
    dv = c.shape[-1]
    out = None if state_only else torch.empty((b, h, n, dv), dtype=bm.dtype, device=DEV)
    st = torch.empty((b, h, dv, dk), dtype=torch.float32, device=DEV) if (want_state or state_only) else None
    nbytes = cuda_lib.lab200_la_workspace_bytes(b * h, n, dk, dv, chunks)
    ws = torch.empty(nbytes, dtype=torch.uint8, device=DEV)
    rc = cuda_lib.lab200_la_generic(
        _lib.ptr(a), bm.data_ptr(), c.data_ptr(), _lib.ptr(s), _lib.ptr(out), _lib.ptr(state_in), _lib.ptr(st),
        ws.data_ptr(), nbytes, b * h, h, n, dk, dv, int(reverse), int(state_only), chunks, _lib.dtype_code(bm.dtype),
        torch.cuda.current_stream().cuda_stream)
    assert rc == 0, cuda_lib.lab200_error_string(rc)
    assert cuda_lib.lab200_read_status(ws.data_ptr(), torch.cuda.current_stream().cuda_stream) == 0
    return out, st


ORACLE_CASES = [
    # b, h, n, dk, dv, reverse, chunks, with_state
    (1, 2, 128, 64, 64, False, 1, False),
    (1, 2, 256, 128, 128, False, 1, True),
    (2, 3, 384, 128, 64, True, 1, True),
    (1, 2, 512, 64, 128, False, 2, True),
    (1, 2, 512, 128, 128, True, 4, True),
    (1, 3, 300, 16, 48, False, 1, False),
    (1, 3, 77, 48, 16, True, 1, False),
    (1, 2, 384, 192, 192, False, 3, True),
    (1, 2, 256, 256, 256, True, 2, True),
    (1, 1, 1, 16, 16, False, 1, False),
    (1, 1, 129, 32, 32, True, 2, False),
    (1, 2, 384, 128, 256, False, 1, True),   # two dv slices per (batch, head) in the pipelined kernel
    (1, 2, 256, 64, 192, True, 2, True),     # dv = 128 + 64: a full and a half-empty slice
]


@pytest.mark.parametrize("b,h,n,dk,dv,reverse,chunks,with_state", ORACLE_CASES)
@pytest.mark.parametrize("slope_scale", [1.0, 0.0])
def test_c_abi_generic_against_numpy_oracle(cuda_lib, b, h, n, dk, dv, reverse, chunks, with_state, slope_scale):
    torch.manual_seed(7)
    a, bm = (torch.randn((b, h, n, dk), device=DEV).bfloat16() for _ in range(2))
    c = torch.randn((b, h, n, dv), device=DEV).bfloat16()
    s = (la._build_slope_tensor(h).reshape(-1) * slope_scale).to(DEV) if slope_scale > 0 else None
    aligned = (n % 128 == 0)
    st_in = torch.randn((b, h, dv, dk), device=DEV) if (with_state and aligned) else None
    out, st = c_generic(cuda_lib, a, bm, c, s, reverse, st_in, aligned, chunks)
    f = lambda t: None if t is None else t.float().cpu().numpy()
    ro, rs = O.la_generic(f(a), f(bm), f(c), f(s), reverse=reverse, state_in=f(st_in))
    assert O.rel_l2_err(f(out), ro) <= 1e-2
    assert O.max_abs_err(f(out), ro) <= 2e-2 * max(1.0, float(np.abs(ro).max()))
    if aligned:
        assert O.rel_l2_err(f(st), rs) <= 1e-2
        # state-only mode returns the same state
        _, st2 = c_generic(cuda_lib, None, bm, c, s, reverse, st_in, True, chunks, state_only=True)
        assert O.rel_l2_err(f(st2), rs) <= 1e-2


@pytest.mark.parametrize("name", ["attn_c1_fp32_sum", "attn_ragged_fp32", "attn_nodecay_fp32", "attn_bf16_div10"])
def test_against_golden_fixtures(cuda_lib, golden_dir, name):
    """Outputs of the reference's torch path (stored fixtures) vs the CUDA path on the same inputs rounded to bf16."""
    g = dict(np.load(os.path.join(golden_dir, name + ".npz")))
    q, k, v = (torch.from_numpy(g[x]).to(DEV).bfloat16().requires_grad_() for x in ("q", "k", "v"))
    do = torch.from_numpy(g["do"]).to(DEV).bfloat16()
    s = torch.from_numpy(g["s"]).to(DEV).reshape(-1, 1, 1) if "s" in g else None
    got = run_fwd_bwd(lambda a, b_, c: la.lightning_attn_func(a, b_, c, s), q, k, v, do)
    scaled = name.endswith("div10")
    for x, key in zip(got, ("o", "dq", "dk", "dv")):
        assert_parity(x, torch.from_numpy(g[key]).to(DEV), f"{name}:{key}", scaled)


def test_chunked_and_serial_sweeps_agree(cuda_lib):
    b, h, n, d = 1, 4, 4096, 128
    q, k, v, _ = make_inputs(b, h, n, d, d, torch.bfloat16, 1.0)
    s = (la._build_slope_tensor(h).reshape(-1) * 0.01).to(DEV)  # slow decay: the carried state matters everywhere
    ref = torch_la_reference(q.detach(), k.detach(), v.detach(), s)
    for chunks in (1, 2, 5, 16):
        out, _ = la_generic(q.detach(), k.detach(), v.detach(), s, chunks=chunks)
        assert_parity(out, ref, f"chunks={chunks}", False)


def test_known_answers_on_gpu(cuda_lib):
    n, d, e = 1000, 16, 16
    q = torch.full((1, 1, n, d), 0.25, device=DEV, dtype=torch.bfloat16)  # 1/sqrt(16)
    v = torch.ones((1, 1, n, e), device=DEV, dtype=torch.bfloat16)
    o = la.lightning_attn_func(q, q, v, None).float()
    # o_t = t + 1 exactly representable in fp32; bf16 output rounding allows 2^-8 relative
    t = torch.arange(1, n + 1, device=DEV, dtype=torch.float32)
    assert float(((o[0, 0, :, 0] - t).abs() / t).max()) <= 2 ** -8
    q1 = torch.zeros((1, 1, n, d), device=DEV, dtype=torch.bfloat16)
    q1[..., 0] = 1
    s = torch.tensor([0.25], device=DEV).reshape(1, 1, 1)
    o = la.lightning_attn_func(q1, q1, q1, s).float()[0, 0, :, 0]
    lam = float(np.exp(-0.25))
    expect = (1 - lam ** t) / (1 - lam)
    assert float(((o - expect).abs() / expect).max()) <= 1e-2


def test_bitwise_determinism(cuda_lib):
    q, k, v, do = make_inputs(2, 4, 1500, 64, 128, torch.bfloat16, 1.0)
    s = la._build_slope_tensor(4).to(DEV)
    r1 = run_fwd_bwd(lambda a, b_, c: la.lightning_attn2(a, b_, c, s), q, k, v, do)
    r2 = run_fwd_bwd(lambda a, b_, c: la.lightning_attn2(a, b_, c, s), q, k, v, do)
    for x, y in zip(r1, r2):
        assert torch.equal(x, y)


@pytest.mark.parametrize("n", [1, 2, 127, 128, 129, 255, 257])
def test_ragged_lengths(cuda_lib, n):
    q, k, v, do = make_inputs(2, 2, n, 32, 64, torch.bfloat16, 1.0)
    s = la._build_slope_tensor(2).to(DEV)
    got = run_fwd_bwd(lambda a, b_, c: la.lightning_attn2(a, b_, c, s), q, k, v, do)
    compare_with_torch_reference(q, k, v, do, s, got, False, f"n={n}")


@pytest.mark.parametrize("d,e", [(24, 40), (16, 16), (96, 80), (160, 208), (256, 256), (320, 64)])
def test_interface_pads_and_splits_feature_dims(cuda_lib, d, e):
    """lightning_attn_func accepts sizes that are not multiples of 16 (zero padding) and d > 256 (feature split),
    the counterpart of the reference's pad/split wrapper (lightning_attn_interface.py:28-63)."""
    q, k, v, do = make_inputs(1, 2, 300, d, e, torch.bfloat16, 1.0)
    s = la._build_slope_tensor(2).to(DEV)
    got = run_fwd_bwd(lambda a, b_, c: la.lightning_attn_func(a, b_, c, s), q, k, v, do)
    assert got[0].shape == (1, 2, 300, e)
    compare_with_torch_reference(q, k, v, do, s, got, False, f"d{d}e{e}")


def test_non_contiguous_inputs_and_no_grad_for_slopes(cuda_lib):
    b, h, n, d = 2, 3, 200, 64
    torch.manual_seed(3)
    qkv = torch.randn((b, n, 3, h, d), device=DEV).bfloat16()
    q, k, v = (qkv[:, :, i].transpose(1, 2).requires_grad_() for i in range(3))  # (b, h, n, d) views
    s = la._build_slope_tensor(h).to(DEV).requires_grad_()
    o = la.lightning_attn_func(q, k, v, s)
    o.sum().backward()
    assert s.grad is None and q.grad is not None
    ref = torch_la_reference(q.detach(), k.detach(), v.detach(), s.detach())
    assert_parity(o, ref, "non-contiguous", False)


@pytest.mark.parametrize("scale", [1.0, 1e-3, 0.0])
def test_sequence_parallel_math_on_one_gpu(cuda_lib, scale):
    """The sequence-parallel scheme run rank by rank on one GPU (no process group): local states from the CUDA
    state-only pass, combined with the package's own `combine_states`, fed back as incoming states, must
    reproduce the unsharded CUDA result and the fp32 reference, forward and backward."""
    from lightning_attention_b200 import distributed as D

    b, h, R, L, d, e = 1, 4, 4, 256, 128, 64
    n = R * L
    q, k, v, do = make_inputs(b, h, n, d, e, torch.bfloat16, 0.5)
    q, k, v = (t.detach() for t in (q, k, v))
    s = (la._build_slope_tensor(h) * scale).to(DEV) if scale > 0 else None
    decay = D._shard_decay(s, h, L, q.device)
    sl = [slice(r * L, (r + 1) * L) for r in range(R)]
    cut = lambda t, r: t[:, :, sl[r]].contiguous()
    fwd_states = [la_generic(None, cut(k, r), cut(v, r), s, state_only=True)[1] for r in range(R)]
    rev_states = [la_generic(None, cut(do, r), cut(q, r), s, reverse=True, state_only=True)[1] for r in range(R)]
    o, dq, dk, dv = [], [], [], []
    for r in range(R):
        kv_in = D.combine_states(fwd_states, decay, r)
        dkv_in = D.combine_states(rev_states, decay, r, reverse=True)
        o.append(la_generic(cut(q, r), cut(k, r), cut(v, r), s, state_in=kv_in)[0])
        dq.append(la_generic(cut(do, r), cut(v, r), cut(k, r), s, state_in=kv_in.transpose(2, 3).contiguous())[0])
        dk.append(la_generic(cut(v, r), cut(do, r), cut(q, r), s, reverse=True, state_in=dkv_in)[0])
        dv.append(la_generic(cut(k, r), cut(q, r), cut(do, r), s, reverse=True,
                             state_in=dkv_in.transpose(2, 3).contiguous())[0])
    got = tuple(torch.cat(x, dim=2) for x in (o, dq, dk, dv))
    qr, kr, vr = (t.float().requires_grad_() for t in (q, k, v))
    ref = run_fwd_bwd(lambda a, b_, c: torch_la_reference(a, b_, c, s), qr, kr, vr, do.float())
    for x, r_, name in zip(got, ref, ("o", "dq", "dk", "dv")):
        assert_parity(x, r_, f"sp-emulated:{name}", False)


@pytest.mark.parametrize("chunks", [1, 3])
@pytest.mark.parametrize("b,h,n,d,e,decay", [(2, 4, 1024, 128, 128, True), (1, 3, 513, 128, 64, True), (2, 2, 300, 64, 128, True),
                                             (1, 2, 77, 32, 16, True), (1, 4, 2048, 128, 128, False), (1, 2, 128, 16, 16, True),
                                             (1, 2, 640, 96, 112, True), (1, 2, 256, 64, 64, True), (1, 1, 384, 128, 128, True)])
def test_fused_dk_dv_sweep(cuda_lib, b, h, n, d, e, decay, chunks):
    """lab200_la2_dkdv (dk and dv in one reverse sweep, one chunk or several) through the C ABI against the fp32 reference
    gradients and against the dk, dv of two launches of the generic kernel."""
    q, k, v, do = make_inputs(b, h, n, d, e, torch.bfloat16, 1.0)
    s = la._build_slope_tensor(h).to(DEV) if decay else None
    sl = None if s is None else s.reshape(-1).contiguous()
    dk = torch.empty_like(k)
    dv = torch.empty_like(v)
    nbytes = cuda_lib.lab200_la_workspace_bytes(b * h, n, e, d, chunks)
    ws = torch.empty(nbytes, dtype=torch.uint8, device=DEV)
    stream = torch.cuda.current_stream().cuda_stream
    rc = cuda_lib.lab200_la2_dkdv(q.data_ptr(), k.data_ptr(), v.data_ptr(), _lib.ptr(sl), do.data_ptr(), dk.data_ptr(),
                                  dv.data_ptr(), None, ws.data_ptr(), nbytes, b, h, n, d, e, chunks, 0, _lib.BF16, stream)
    assert rc == 0, cuda_lib.lab200_error_string(rc)
    assert cuda_lib.lab200_read_status(ws.data_ptr(), stream) == 0
    qr, kr, vr = (t.detach().float().requires_grad_() for t in (q, k, v))
    _, _, rdk, rdv = run_fwd_bwd(lambda a, b_, c: torch_la_reference(a, b_, c, s), qr, kr, vr, do.float())
    assert_parity(dk, rdk, "fused:dk", False)
    assert_parity(dv, rdv, "fused:dv", False)
    gdk, _ = la_generic(v.detach(), do, q.detach(), s, reverse=True, chunks=chunks)
    gdv, _ = la_generic(k.detach(), q.detach(), do, s, reverse=True, chunks=chunks)
    assert_parity(dk, gdk.float(), "fused-vs-generic:dk", False)
    assert_parity(dv, gdv.float(), "fused-vs-generic:dv", False)


@pytest.mark.parametrize("b,h,n", [(2, 8, 4096), (4, 32, 1024)])  # few pairs: sequences cut into chunks; 128 pairs: one sweep per pair
def test_block_kernels_are_deterministic(cuda_lib, b, h, n):
    """Five runs of forward + backward on the same inputs give bit-identical o, dq, dk, dv: the hand-overs between the roles of
    the block kernels (mbarriers, TMEM and shared-memory reuse) leave no window in which a tile is read early or late."""
    q, k, v, do = make_inputs(b, h, n, 128, 128, torch.bfloat16, 1.0)
    s = la._build_slope_tensor(h).to(DEV)
    ref = None
    for _ in range(5):
        qq, kk, vv = (t.detach().clone().requires_grad_() for t in (q, k, v))
        o = la.lightning_attn2(qq, kk, vv, s)
        o.backward(do)
        torch.cuda.synchronize()
        got = tuple(t.detach().view(torch.int16).clone() for t in (o, qq.grad, kk.grad, vv.grad))
        if ref is None:
            ref = got
        else:
            for a, b_, name in zip(got, ref, ("o", "dq", "dk", "dv")):
                assert torch.equal(a, b_), f"{name} differs between runs"


@pytest.mark.parametrize("chunks", [1, 2])
@pytest.mark.parametrize("scale", [1.0, 1e-2])
def test_fused_dk_dv_with_incoming_state_and_kept_chunk_states(cuda_lib, chunks, scale):
    """The sequence-parallel use of the fused sweep: the second half of a sequence, given the reverse-time state that its
    (absent) continuation contributes, equals the matching rows of the whole sequence; with and without the two-step
    protocol that reuses the chunk states of a state-only call on (do, q)."""
    b, h, n, d, e = 1, 4, 1024, 128, 64
    q, k, v, do = (t.detach() for t in make_inputs(b, h, n, d, e, torch.bfloat16, 1.0, seed=11))
    s = la._build_slope_tensor(h).to(DEV) * scale
    whole_dk, whole_dv = la.la_dkdv(q, k, v, s, do)
    half = n // 2
    lo = lambda t: t[:, :, :half].contiguous()
    hi = lambda t: t[:, :, half:].contiguous()
    _, tail_state = la_generic(None, hi(do), hi(q), s, reverse=True, state_only=True)  # (b, h, d, e): what tokens >= half contribute
    dk1, dv1 = la.la_dkdv(lo(q), lo(k), lo(v), s, lo(do), state_in=tail_state, chunks=chunks)
    do_lo, q_lo = lo(do), lo(q)
    _, _, handle = la_generic(None, do_lo, q_lo, s, reverse=True, state_only=True, keep_workspace=True, chunks=chunks)
    dk2, dv2 = la.la_dkdv(q_lo, lo(k), lo(v), s, do_lo, state_in=tail_state, chunks=chunks, resume_from=handle)
    for got_k, got_v, tag in ((dk1, dv1, "direct"), (dk2, dv2, "resumed")):
        assert_parity(got_k, whole_dk[:, :, :half].float(), f"fused-state-{tag}:dk", False)
        assert_parity(got_v, whole_dv[:, :, :half].float(), f"fused-state-{tag}:dv", False)


def test_fused_dk_dv_reads_and_writes_the_projection_layout(cuda_lib):
    """(b, n, h, dim) tensors in place: bit-identical to the default layout."""
    b, h, n, d, e = 2, 4, 640, 128, 128
    q, k, v, do = (t.detach() for t in make_inputs(b, h, n, d, e, torch.bfloat16, 1.0, seed=12))
    s = la._build_slope_tensor(h).to(DEV)
    dk, dv = la.la_dkdv(q, k, v, s, do)
    view = lambda t: t.transpose(1, 2).contiguous().transpose(1, 2)  # same values, (b, n, h, dim) storage
    dk2, dv2 = la.la_dkdv(view(q), view(k), view(v), s, view(do))
    assert dk2.stride() == view(q).stride() and dv2.stride() == view(v).stride()
    assert torch.equal(dk2, dk) and torch.equal(dv2, dv)


@pytest.mark.parametrize("reverse", [False, True])
@pytest.mark.parametrize("chunks", [1, 3])
def test_two_step_generic_call_reuses_chunk_states(cuda_lib, reverse, chunks):
    """state-only call + lab200_la_generic_resume with an incoming state == one call with that state."""
    torch.manual_seed(9)
    b, h, n, dk, dv = 1, 3, 1536, 128, 64
    a, bm = (torch.randn((b, h, n, dk), device=DEV).bfloat16() for _ in range(2))
    c = torch.randn((b, h, n, dv), device=DEV).bfloat16()
    s = (la._build_slope_tensor(h).reshape(-1) * 0.02).to(DEV)
    st_in = torch.randn((b, h, dv, dk), device=DEV)
    ref, _ = la_generic(a, bm, c, s, reverse=reverse, state_in=st_in, chunks=chunks)
    _, st_loc, handle = la_generic(None, bm, c, s, reverse=reverse, state_only=True, chunks=chunks, keep_workspace=True)
    got, _ = la_generic(a, bm, c, s, reverse=reverse, state_in=st_in, chunks=chunks, resume_from=handle)
    assert_parity(got, ref.float(), "two-step", False)
    _, st_loc2 = la_generic(None, bm, c, s, reverse=reverse, state_only=True, chunks=chunks)
    assert torch.equal(st_loc, st_loc2)


@pytest.mark.parametrize("reverse", [False, True])
@pytest.mark.parametrize("chunks", [1, 3])
@pytest.mark.parametrize("d", [128, 48])
def test_swapped_resume_reuses_transposed_chunk_states(cuda_lib, reverse, chunks, d):
    """The chunk states of the product on (bm, c) serve the product on (c, bm) after an in-place transpose
    (lab200_la_generic_resume_swapped): from a state-only call (incoming state still to be added) and from a resumed
    call (incoming state already in)."""
    torch.manual_seed(10)
    b, h, n = 1, 3, 1536
    a, bm, c, a2 = (torch.randn((b, h, n, d), device=DEV).bfloat16() for _ in range(4))
    s = (la._build_slope_tensor(h).reshape(-1) * 0.02).to(DEV)
    st_in = torch.randn((b, h, d, d), device=DEV)
    st_in_t = st_in.transpose(2, 3).contiguous()
    ref_swapped, _ = la_generic(a2, c, bm, s, reverse=reverse, state_in=st_in_t, chunks=chunks)
    # state-only on (bm, c) -> swapped resume on (c, bm), which adds the incoming state itself
    _, _, handle = la_generic(None, bm, c, s, reverse=reverse, state_only=True, chunks=chunks, keep_workspace=True)
    got, _ = la_generic(a2, c, bm, s, reverse=reverse, state_in=st_in_t, chunks=chunks, resume_from=handle, resume_swapped=True)
    assert_parity(got, ref_swapped.float(), "swapped-from-state-only", False)
    # state-only -> resume on (bm, c) with the incoming state -> swapped resume on (c, bm) without adding it again
    ref, _ = la_generic(a, bm, c, s, reverse=reverse, state_in=st_in, chunks=chunks)
    _, _, handle = la_generic(None, bm, c, s, reverse=reverse, state_only=True, chunks=chunks, keep_workspace=True)
    got, _, handle = la_generic(a, bm, c, s, reverse=reverse, state_in=st_in, chunks=chunks, resume_from=handle, keep_workspace=True)
    assert_parity(got, ref.float(), "resumed", False)
    got, _ = la_generic(a2, c, bm, s, reverse=reverse, state_in=st_in_t, chunks=chunks, resume_from=handle,
                        resume_swapped=True, rebase=False)
    assert_parity(got, ref_swapped.float(), "swapped-from-resumed", False)
    with pytest.raises(RuntimeError):  # the handle now belongs to (c, bm)
        la_generic(a2, c, bm, s, reverse=reverse, chunks=chunks, resume_from=handle, resume_swapped=True)


@pytest.mark.parametrize("chunks", [0, 5])
@pytest.mark.parametrize("d", [128, 64, 192])
def test_chunked_backward_shares_chunk_states_between_dk_and_dv(cuda_lib, chunks, d):
    """Few (batch, head) pairs and d == e: lab200_la2_bwd runs in chunk mode and dv takes dk's chunk states transposed."""
    from lightning_attention_b200.ops.cuda.lightning_attn2 import _bwd, _fwd, _slopes_arg

    b, h, n = 1, 4, 4096 + 128 * 3
    q, k, v, do = make_inputs(b, h, n, d, d, torch.bfloat16, 1.0, seed=77)
    s = (la._build_slope_tensor(h).reshape(-1) * 0.01).to(DEV)  # slow decay: the carried state matters everywhere
    sl = _slopes_arg(s, h, q.device)
    with torch.no_grad():
        o = _fwd(q, k, v, sl, chunks=chunks)
        dq, dk, dv = _bwd(q, k, v, sl, do, chunks=chunks)
    compare_with_torch_reference(q, k, v, do, s, (o, dq, dk, dv), False, f"chunked-bwd-d{d}-c{chunks}")


@pytest.mark.parametrize("x,y", [(128, 128), (48, 80), (16, 200)])
@pytest.mark.parametrize("decay", [True, False])
def test_combine_states_kernel_matches_formula(cuda_lib, x, y, decay):
    """lab200_la_combine_states == the torch formula of distributed.combine_states, both layouts, every rank, both directions."""
    from lightning_attention_b200 import distributed as D

    torch.manual_seed(3)
    R, b, h, L = 5, 2, 3, 256
    gathered = torch.randn((R, b, h, x, y), device=DEV)
    s = (la._build_slope_tensor(h).reshape(-1) * 0.01).to(DEV) if decay else None
    dec = D._shard_decay(s, h, L, gathered.device)
    for rank in range(R):
        for reverse in (False, True):
            ref = D.combine_states(gathered, dec, rank, reverse=reverse)
            got, got_t = D.combine_gathered(gathered, s, L, rank, reverse=reverse)
            assert torch.allclose(got, ref, rtol=1e-5, atol=1e-5), (rank, reverse)
            assert torch.equal(got_t, got.transpose(2, 3).contiguous())


@pytest.mark.parametrize("decay", [True, False])
def test_autograd_in_chunk_mode_hands_chunk_states_from_forward_to_backward(cuda_lib, decay):
    """Few (batch, head) pairs, d == e: the autograd Function keeps the forward's chunk states for dq and dk's for dv.
    A second backward through the same graph (states already handed over) must give the same gradients."""
    b, h, n, d = 1, 4, 4096 + 128 * 3, 128
    assert cuda_lib.lab200_la_plan_chunks(b * h, n, d, d) > 1
    q, k, v, do = make_inputs(b, h, n, d, d, torch.bfloat16, 1.0 if decay else 0.2, seed=78)
    s = (la._build_slope_tensor(h).reshape(-1) * 0.01).to(DEV) if decay else None
    o = la.lightning_attn_func(q, k, v, s)
    o.backward(do, retain_graph=True)
    first = tuple(t.grad.clone() for t in (q, k, v))
    q.grad = k.grad = v.grad = None
    o.backward(do)
    second = (q.grad, k.grad, v.grad)
    compare_with_torch_reference(q, k, v, do, s, (o.detach(),) + first, False, f"autograd-chunked-decay{decay}")
    for x, y in zip(first, second):
        assert_parity(x, y.float(), "second-backward", False)


@pytest.mark.parametrize("n,dk,dv,chunks", [(300, 64, 64, 1), (171, 128, 128, 1), (1000, 128, 64, 3), (77, 192, 192, 1), (129, 32, 48, 2)])
@pytest.mark.parametrize("slope_scale", [1.0, 0.05, 0.0])
def test_forward_state_out_is_exact_for_ragged_lengths(cuda_lib, n, dk, dv, chunks, slope_scale):
    """state_out of a forward-time call is the state entering token n for any n: checked against the definition
    (oracle.state_entering), with and without an incoming state, in one sweep and in chunk mode."""
    torch.manual_seed(21)
    b, h = 1, 3
    a, bm = (torch.randn((b, h, n, dk), device=DEV).bfloat16() for _ in range(2))
    c = torch.randn((b, h, n, dv), device=DEV).bfloat16()
    s = (la._build_slope_tensor(h).reshape(-1) * slope_scale).to(DEV) if slope_scale > 0 else None
    f = lambda t: None if t is None else t.float().cpu().numpy()
    for st_in in (None, torch.randn((b, h, dv, dk), device=DEV)):
        _, st = c_generic(cuda_lib, a, bm, c, s, False, st_in, True, chunks)
        ref = O.state_entering(f(bm), f(c), f(s), state_in=f(st_in))
        assert O.rel_l2_err(f(st), ref) <= 1e-2, (n, dk, dv, chunks, st_in is not None)
        st_only = c_generic(cuda_lib, None, bm, c, s, False, st_in, True, chunks, state_only=True)[1]
        assert O.rel_l2_err(f(st_only), ref) <= 1e-2


@pytest.mark.parametrize("d,e", [(128, 128), (64, 96), (192, 192)])
@pytest.mark.parametrize("decay", [True, False])
def test_prefill_chunks_and_decode_steps_continue_the_sequence(cuda_lib, d, e, decay):
    """prefill(0..n1) -> prefill(n1..n2, state) -> decode steps == one forward over the whole sequence."""
    torch.manual_seed(22)
    b, h, n, n1, n2 = 2, 4, 700, 300, 684
    q, k = (torch.randn((b, h, n, d), device=DEV).bfloat16() for _ in range(2))
    v = torch.randn((b, h, n, e), device=DEV).bfloat16()
    s = (la._build_slope_tensor(h) * 0.2).to(DEV) if decay else None
    ref = torch_la_reference(q, k, v, s)
    o1, st = la.lightning_attn_prefill(q[:, :, :n1].contiguous(), k[:, :, :n1].contiguous(), v[:, :, :n1].contiguous(), s)
    o2, st = la.lightning_attn_prefill(q[:, :, n1:n2].contiguous(), k[:, :, n1:n2].contiguous(), v[:, :, n1:n2].contiguous(), s, st)
    outs = [o1, o2]
    for t in range(n2, n):
        outs.append(la.lightning_attn_decode(q[:, :, t:t + 1], k[:, :, t:t + 1], v[:, :, t:t + 1], s, st))
    got = torch.cat(outs, dim=2)
    assert_parity(got, ref, f"prefill+decode d{d} e{e}", False)
    assert_parity(got[:, :, n2:], ref[:, :, n2:], "decode steps", False)
    f = lambda t: None if t is None else t.float().cpu().numpy()
    assert O.rel_l2_err(f(st), O.state_entering(f(k), f(v), f(s))) <= 1e-2


def test_decode_step_against_numpy_oracle(cuda_lib):
    torch.manual_seed(23)
    b, h, d, e = 3, 5, 48, 80
    q, k = (torch.randn((b, h, d), device=DEV).half() for _ in range(2))
    v = torch.randn((b, h, e), device=DEV).half()
    st = torch.randn((b, h, e, d), device=DEV)
    s = la._build_slope_tensor(h).to(DEV)
    f = lambda t: t.float().cpu().numpy()
    ro, rst = O.decode_step(f(q), f(k), f(v), f(s), f(st))
    o = la.lightning_attn_decode(q, k, v, s, st)
    assert O.rel_l2_err(f(o), ro) <= 2e-3
    assert O.rel_l2_err(f(st), rst) <= 1e-6
    with pytest.raises(RuntimeError):
        la.lightning_attn_decode(q, k, v, s, st.transpose(2, 3))


@pytest.mark.parametrize("b,h,n,d,e", [(4, 32, 512, 128, 128), (1, 4, 4096, 128, 128), (2, 3, 300, 64, 96), (1, 8, 2048, 128, 64),
                                       (2, 12, 384, 192, 192)])
@pytest.mark.parametrize("decay", [True, False])
def test_projection_layout_is_read_and_written_in_place(cuda_lib, b, h, n, d, e, decay):
    """q, k, v given as (b, h, n, d) views of (b, n, h, d) tensors - what rearranging a projection output gives
    (examples/module/tnl_attn.py:56-59) - are read in place and o, dq, dk, dv come back in the same layout, with exactly
    the values of the contiguous path (d > 128 falls back to copies and must still agree)."""
    from lightning_attention_b200.ops.cuda.lightning_attn2 import _is_bnhd

    torch.manual_seed(31)
    xq, xk = (torch.randn((b, n, h, d), device=DEV).bfloat16().requires_grad_() for _ in range(2))
    xv = torch.randn((b, n, h, e), device=DEV).bfloat16().requires_grad_()
    xdo = torch.randn((b, n, h, e), device=DEV).bfloat16()
    s = la._build_slope_tensor(h).to(DEV) if decay else None
    o = la.lightning_attn_func(xq.transpose(1, 2), xk.transpose(1, 2), xv.transpose(1, 2), s)
    o.backward(xdo.transpose(1, 2))
    if max(d, e) <= 128:
        assert _is_bnhd(o) and o.transpose(1, 2).is_contiguous()
    q, k, v = (t.detach().transpose(1, 2).contiguous().requires_grad_() for t in (xq, xk, xv))
    ro = la.lightning_attn_func(q, k, v, s)
    ro.backward(xdo.transpose(1, 2).contiguous())
    assert torch.equal(o, ro)
    for x, r, name in ((xq, q, "dq"), (xk, k, "dk"), (xv, v, "dv")):
        assert torch.equal(x.grad.transpose(1, 2), r.grad), name
    compare_with_torch_reference(q, k, v, xdo.transpose(1, 2).contiguous(), s,
                                 (o.detach(), xq.grad.transpose(1, 2), xk.grad.transpose(1, 2), xv.grad.transpose(1, 2)), False,
                                 f"bnhd-{b}-{h}-{n}-{d}-{e}")


def test_projection_layout_through_the_c_abi(cuda_lib):
    """lab200_la_generic with LAB200_LAYOUT_BNHD: forward and reverse time, with states, against the default layout."""
    torch.manual_seed(32)
    b, h, n, dk, dv = 2, 3, 640, 64, 128
    xa, xb = (torch.randn((b, n, h, dk), device=DEV).bfloat16() for _ in range(2))
    xc = torch.randn((b, n, h, dv), device=DEV).bfloat16()
    s = (la._build_slope_tensor(h).reshape(-1) * 0.05).to(DEV)
    st_in = torch.randn((b, h, dv, dk), device=DEV)
    for reverse in (False, True):
        for chunks in (1, 3):
            got, gst = la_generic(xa.transpose(1, 2), xb.transpose(1, 2), xc.transpose(1, 2), s, reverse=reverse, state_in=st_in,
                                  want_state=True, chunks=chunks)
            ref, rst = la_generic(xa.transpose(1, 2).contiguous(), xb.transpose(1, 2).contiguous(), xc.transpose(1, 2).contiguous(),
                                  s, reverse=reverse, state_in=st_in, want_state=True, chunks=chunks)
            assert got.transpose(1, 2).is_contiguous()
            assert torch.equal(got, ref) and torch.equal(gst, rst), (reverse, chunks)


def _random_case(seed):
    rng = np.random.default_rng(1000 + seed)
    b = int(rng.integers(1, 4))
    h = int(rng.integers(1, 6))
    n = int(rng.integers(1, 900))
    dk = 16 * int(rng.integers(1, 17))
    dv = 16 * int(rng.integers(1, 17))
    reverse = bool(rng.integers(0, 2))
    chunks = int(rng.choice([0, 1, 2, 5]))
    layout = bool(rng.integers(0, 2)) and dk <= 128 and dv <= 128
    with_state = bool(rng.integers(0, 2)) and not (reverse and n % 128)
    slope_scale = float(rng.choice([0.0, 0.02, 1.0]))
    return b, h, n, dk, dv, reverse, chunks, layout, with_state, slope_scale


@pytest.mark.parametrize("seed", range(32))
def test_randomised_shapes_against_numpy_oracle(cuda_lib, seed):
    """Seeded random draws over batch, heads, length, feature dims (16..256), direction, chunking, layout, incoming state
    and decay strength; output and outgoing state against the numpy oracle."""
    b, h, n, dk, dv, reverse, chunks, layout, with_state, slope_scale = _random_case(seed)
    torch.manual_seed(seed)
    if layout:
        a, bm = (torch.randn((b, n, h, dk), device=DEV).bfloat16().transpose(1, 2) for _ in range(2))
        c = torch.randn((b, n, h, dv), device=DEV).bfloat16().transpose(1, 2)
    else:
        a, bm = (torch.randn((b, h, n, dk), device=DEV).bfloat16() for _ in range(2))
        c = torch.randn((b, h, n, dv), device=DEV).bfloat16()
    s = (la._build_slope_tensor(h).reshape(-1) * slope_scale).to(DEV) if slope_scale > 0 else None
    st_in = torch.randn((b, h, dv, dk), device=DEV) if with_state else None
    want_state = (not reverse) or n % 128 == 0
    out, st = la_generic(a, bm, c, s, reverse=reverse, state_in=st_in, want_state=want_state, chunks=chunks)
    f = lambda t: None if t is None else t.float().cpu().numpy()
    ro, rs = O.la_generic(f(a), f(bm), f(c), f(s), reverse=reverse, state_in=f(st_in))
    tag = str(_random_case(seed))
    assert O.rel_l2_err(f(out), ro) <= 1e-2, tag
    assert O.max_abs_err(f(out), ro) <= 2e-2 * max(1.0, float(np.abs(ro).max())), tag
    if want_state:
        assert O.rel_l2_err(f(st), rs) <= 1e-2, tag


# ------------------------------------------------------------------------------------------------------------------
# long sequences where the running state never dies out (no decay, very slow decay): error growth with n
# ------------------------------------------------------------------------------------------------------------------
LONG_N_RESULTS = {}


@pytest.mark.parametrize("variant", ["no_decay", "slopes_x1e-3", "alibi"])
@pytest.mark.parametrize("n", [2048, 8192, 32768, 131072])
def test_long_sequences_with_a_state_that_never_dies(cuda_lib, n, variant):
    """b1 h4 d=e=128 bf16, q, k, v ~ 0.5 N(0,1): no decay, ALiBi slopes x 1e-3 and ALiBi slopes at n up to 131072 (chunk mode:
    4 pairs on 148 SMs) against the fp32 block recurrence. The state is carried in fp32 but fed to the tensor cores as a
    bf16 copy, so this is where a rounding error that grows with n would show."""
    b, h, d = 1, 4, 128
    q, k, v, do = make_inputs(b, h, n, d, d, torch.bfloat16, 0.5, seed=31)
    s = None if variant == "no_decay" else la._build_slope_tensor(h).to(DEV) * (1e-3 if variant == "slopes_x1e-3" else 1.0)
    fn = (lambda a, b_, c: la.lightning_attn2_no_decay(a, b_, c)) if s is None else (lambda a, b_, c: la.lightning_attn2(a, b_, c, s))
    got = run_fwd_bwd(fn, q, k, v, do)
    qr, kr, vr = (t.detach().float().requires_grad_() for t in (q, k, v))
    ref = run_fwd_bwd(lambda a, b_, c: torch_la_reference(a, b_, c, s), qr, kr, vr, do.float())
    rels = {}
    for x, r, name in zip(got, ref, ("o", "dq", "dk", "dv")):
        rels[name] = errs(x, r)[1]
        assert_parity(x, r, f"long-{variant}-n{n}:{name}", False)
    LONG_N_RESULTS[(variant, n)] = rels
    print(f"rel-L2 {variant} n={n}: " + " ".join(f"{k_}={v_:.2e}" for k_, v_ in rels.items()))


def test_backward_with_unequal_feature_dims_in_chunk_mode(cuda_lib):
    """d != e with few (batch, head) pairs: the three products of the backward pass plan different chunk counts and the
    workspace must cover the largest (lab200_la2_bwd_workspace_bytes)."""
    for (b, h, n, d, e) in ((1, 32, 2048, 128, 256), (1, 32, 2048, 64, 192)):
        q, k, v, do = make_inputs(b, h, n, d, e, torch.bfloat16, 1.0, seed=5)
        s = la._build_slope_tensor(h).to(DEV)
        got = run_fwd_bwd(lambda a, b_, c: la.lightning_attn2(a, b_, c, s), q, k, v, do)
        compare_with_torch_reference(q, k, v, do, s, got, False, f"unequal-dims{(d, e)}")


def test_interface_splits_wide_value_dims(cuda_lib):
    """e > 256 through lightning_attn_func: column slices of v, forward and backward (the reference pads e to a power of
    two instead, lightning_attn_interface.py:28-32)."""
    b, h, n, d, e = 1, 2, 384, 64, 320
    q, k, v, do = make_inputs(b, h, n, d, e, torch.bfloat16, 1.0, seed=6)
    s = la._build_slope_tensor(h).to(DEV)
    got = run_fwd_bwd(lambda a, b_, c: la.lightning_attn_func(a, b_, c, s), q, k, v, do)
    assert got[0].shape == (b, h, n, e)
    compare_with_torch_reference(q, k, v, do, s, got, False, "wide-e")


def test_fp32_inputs_are_refused_with_a_clear_message(cuda_lib):
    q = torch.randn(1, 2, 128, 64, device=DEV)
    with pytest.raises(RuntimeError, match="bf16 or fp16"):
        la.lightning_attn2(q, q, q, la._build_slope_tensor(2).to(DEV))


def test_expired_device_wait_reaches_the_caller_one_call_late(cuda_lib):
    """The bounded waits of the block kernels end in an error word, not a hang. Here a tiny kernel lets such a wait run out
    on purpose (a barrier nothing arrives on, 1e5-cycle budget, no copies or MMAs in flight); the word must show up in the
    workspace, then through lab200_last_status, and the next operator call must raise - after which the device is usable."""
    ws = torch.zeros(256, dtype=torch.uint8, device=DEV)
    stream = torch.cuda.current_stream().cuda_stream
    torch.cuda.synchronize()
    assert cuda_lib.lab200_last_status() == 0
    assert cuda_lib.lab200_debug_wait_expiry(ws.data_ptr(), 256, 100000, stream) == 0
    assert cuda_lib.lab200_read_status(ws.data_ptr(), stream) == 101  # synchronises
    torch.cuda.synchronize()
    q, k, v, _ = make_inputs(1, 2, 256, 64, 64, torch.bfloat16, 1.0)
    s = la._build_slope_tensor(2).to(DEV)
    with pytest.raises(RuntimeError, match="earlier lightning attention call"):
        la.lightning_attn2(q, k, v, s)
    assert cuda_lib.lab200_last_status() == 0  # reported once
    o = la.lightning_attn2(q, k, v, s)  # the context is intact
    torch.cuda.synchronize()
    assert torch.isfinite(o.float()).all()
    assert cuda_lib.lab200_last_status() == 0
