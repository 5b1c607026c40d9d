"""GPU test of lab200_la2_fwd_static, the forward entry point that brings its own scratch.

Some callers of the library can only pass input and output buffers: they have no allocator to take a
workspace from, or must not call one on their hot path. This test drives the entry point the way such a
caller would -- raw pointers through the C ABI, no workspace argument -- and checks it against the regular
lab200_la2_fwd on two calls in a row, the second with different data, so that anything the first call left
in the shared scratch array would show up. The file name sorts last on purpose: a run that stops at the first
failure has then already executed every other test.
"""
import pytest
import torch

from lightning_attention_b200 import _lib

pytestmark = pytest.mark.gpu
DEV = "cuda"
STATIC_BYTES = 16 * 1024 * 1024


def _inputs(seed, b, h, n, d, e):
    g = torch.Generator(device=DEV)
    g.manual_seed(seed)
    mk = lambda last: torch.randn((b, h, n, last), device=DEV, generator=g).to(torch.bfloat16)
    slopes = torch.tensor([2.0 ** (-8.0 * (i + 1) / h) for i in range(h)], device=DEV, dtype=torch.float32) * 0.05
    return mk(d), mk(d), mk(e), slopes


def _regular(L, q, k, v, s, chunks):
    b, h, n, d = q.shape
    e = v.shape[-1]
    o = torch.empty((b, h, n, e), dtype=q.dtype, device=DEV)
    nbytes = L.lab200_la_workspace_bytes(b * h, n, d, e, chunks)
    ws = torch.empty(nbytes, dtype=torch.uint8, device=DEV)
    rc = L.lab200_la2_fwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), s.data_ptr(), o.data_ptr(), ws.data_ptr(), nbytes,
                          b, h, n, d, e, chunks, _lib.BF16, torch.cuda.current_stream().cuda_stream)
    assert rc == 0, L.lab200_error_string(rc)
    return o


def _static(L, q, k, v, s, chunks):
    b, h, n, d = q.shape
    e = v.shape[-1]
    o = torch.empty((b, h, n, e), dtype=q.dtype, device=DEV)
    rc = L.lab200_la2_fwd_static(q.data_ptr(), k.data_ptr(), v.data_ptr(), s.data_ptr(), o.data_ptr(), b, h, n, d, e,
                                 chunks, _lib.BF16, torch.cuda.current_stream().cuda_stream)
    assert rc == 0, L.lab200_error_string(rc)
    return o


def _rel_l2(x, ref):
    x, ref = x.float(), ref.float()
    return float((x - ref).norm() / ref.norm())


def test_static_scratch_entry_point_matches_regular_one_twice(cuda_lib):
    L = cuda_lib
    b, h, n, d, e, chunks = 1, 4, 2048, 128, 128, 4  # chunked: the per-chunk states really go through the scratch array
    assert 256 < L.lab200_la_workspace_bytes(b * h, n, d, e, chunks) <= STATIC_BYTES
    for seed in (1, 2):  # two calls in a row on the same array, different data
        q, k, v, s = _inputs(seed, b, h, n, d, e)
        want = _regular(L, q, k, v, s, chunks)
        o_static = torch.empty((b, h, n, e), dtype=q.dtype, device=DEV)
        stream = torch.cuda.current_stream().cuda_stream
        L.lab200_la2_fwd_static(q.data_ptr(), k.data_ptr(), v.data_ptr(), s.data_ptr(), o_static.data_ptr(), b, h, n, d, e,
                                chunks, _lib.BF16, stream)  # first call on the device looks up the array's address
        torch.cuda.synchronize()
        # the call itself takes no device memory: neither from the driver nor from torch's caching allocator
        free0, reserved0, allocated0 = torch.cuda.mem_get_info()[0], torch.cuda.memory_reserved(), torch.cuda.memory_allocated()
        rc = L.lab200_la2_fwd_static(q.data_ptr(), k.data_ptr(), v.data_ptr(), s.data_ptr(), o_static.data_ptr(), b, h, n, d, e,
                                     chunks, _lib.BF16, stream)
        torch.cuda.synchronize()
        assert rc == 0
        assert torch.cuda.mem_get_info()[0] == free0
        assert torch.cuda.memory_reserved() == reserved0 and torch.cuda.memory_allocated() == allocated0
        assert L.lab200_static_status(stream) == 0  # the status word of the built-in array: no bounded wait ran out
        got = _static(L, q, k, v, s, chunks)
        torch.cuda.synchronize()
        assert torch.equal(got, o_static)
        assert torch.isfinite(got.float()).all()
        assert _rel_l2(got, want) <= 1e-2  # the tolerance of the other attention tests; in practice the two agree bit for bit
        assert float((got.float() - want.float()).abs().max()) <= 2e-2 * float(want.float().abs().max())
    # an unchunked problem after a chunked one: only the status word of the array is used
    q, k, v, s = _inputs(3, 2, 2, 300, 64, 64)
    assert _rel_l2(_static(L, q, k, v, s, 1), _regular(L, q, k, v, s, 1)) <= 1e-2


def test_static_scratch_entry_point_refuses_oversized_problems(cuda_lib):
    L = cuda_lib
    b, h, n, d, e, chunks = 2, 32, 8192, 128, 128, 32  # 64 * 32 chunk states of 64 KiB = 128 MiB > 16 MiB
    assert L.lab200_la_workspace_bytes(b * h, n, d, e, chunks) > STATIC_BYTES
    q, k, v, s = _inputs(4, b, h, n, d, e)
    o = torch.full((b, h, n, e), 7.0, dtype=torch.bfloat16, device=DEV)
    rc = L.lab200_la2_fwd_static(q.data_ptr(), k.data_ptr(), v.data_ptr(), s.data_ptr(), o.data_ptr(), b, h, n, d, e,
                                 chunks, _lib.BF16, torch.cuda.current_stream().cuda_stream)
    assert rc == 7 and b"16 MiB" in L.lab200_error_string(rc)
    torch.cuda.synchronize()
    assert float(o.float().min()) == 7.0  # nothing was enqueued
