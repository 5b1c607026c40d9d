"""torch.autograd.Functions for Lightning Attention-2 backed by liblightning_b200.so.

Mirrors the operator layer of the reference: ``LightningAttention2`` / ``lightning_attn2``
(lightning_attn/ops/triton/lightning_attn2.py:398-507) and ``LightningAttention2NoDecay`` /
``lightning_attn2_no_decay`` (lightning_attn2_no_decay.py:367-471). Inputs are made contiguous,
outputs are allocated here with torch, (q, k, v, s) are saved for backward, and ``s`` receives no
gradient, exactly as there. All device work goes through the C ABI on the current CUDA stream.
"""
import torch

from ... import _lib


def _slopes_arg(s, h, device):
    """First h entries of `s` as contiguous fp32 on `device` (the reference kernels read S + head index,
    lightning_attn2.py:26,39-42), or None."""
    if s is None:
        return None
    flat = s.detach().to(device=device, dtype=torch.float32).contiguous().view(-1)
    if flat.numel() < h:
        raise RuntimeError(f"slope tensor has {flat.numel()} entries, need at least h={h}")
    return flat[:h].contiguous()


LAYOUT_BNHD = 0x100  # LAB200_LAYOUT_BNHD


def _is_bnhd(t):
    """True if the (b, h, n, d) tensor is a view of a contiguous (b, n, h, d) one - what
    `rearrange(x, "b n (h d) -> b h n d")` of a projection output gives (examples/module/tnl_attn.py:56-59)."""
    if t is None or t.dim() != 4:
        return False
    b, h, n, d = t.shape
    return h > 1 and n > 1 and t.stride() == (n * h * d, d, h * d, 1) and t.data_ptr() % 16 == 0


def _empty_bnhd(b, h, n, d, dtype, device):
    return torch.empty((b, n, h, d), dtype=dtype, device=device).transpose(1, 2)


def _to_layout(t, bnhd):
    """`t` in the layout the call uses: as is when it already has it, else one copy."""
    if not bnhd:
        return t.contiguous()
    if _is_bnhd(t):
        return t
    b, h, n, d = t.shape
    return _empty_bnhd(b, h, n, d, t.dtype, t.device).copy_(t)


def _use_bnhd(*tensors):
    """The library reads (b, n, h, dim) tensors in place when every tensor of the call has that layout and all feature
    dims are <= 128 (the pipelined kernel); anything else is made (b, h, n, dim) contiguous first, as the reference does."""
    return all(_is_bnhd(t) for t in tensors) and all(t.shape[-1] <= 128 and t.shape[-1] % 16 == 0 for t in tensors)


def _empty_out(b, h, n, d, dtype, device, bnhd):
    return _empty_bnhd(b, h, n, d, dtype, device) if bnhd else torch.empty((b, h, n, d), dtype=dtype, device=device)


def _workspace(nbytes, device):
    return torch.empty(int(nbytes), dtype=torch.uint8, device=device)


class KeptWorkspace:
    """Workspace of a chunked product kept for a later resume: the buffer, the product it belongs to (sizes, options and
    the addresses of bm and c) and whether the state entering the sequence is already part of its chunk states."""
    __slots__ = ("ws", "nbytes", "key", "based")

    def __init__(self, ws, nbytes, key, based):
        self.ws, self.nbytes, self.key, self.based = ws, nbytes, key, based


def _product_key(bm, c, reverse, chunks):
    b, h, n, dk = bm.shape
    return (b, h, n, dk, c.shape[-1], bool(reverse), int(chunks), bm.dtype, bm.data_ptr(), c.data_ptr(), bm.stride(), c.stride())


def la_generic(a, bm, c, s=None, reverse=False, state_in=None, want_state=False, state_only=False, chunks=0,
               keep_workspace=False, resume_from=None, resume_swapped=False, rebase=True):
    """The decayed causal product all attention results are instances of (see include/lightning_b200.h).

    a, bm: (b, h, n, dk); c: (b, h, n, dv). Returns (out, state_out) with out (b, h, n, dv) in the
    input dtype (None when state_only) and state_out (b, h, dv, dk) fp32 (None unless requested).
    state_in, if given, has the shape of state_out and is the running state entering the sequence.

    Two-step use (sequence parallelism): call with state_only=True, keep_workspace=True -> (None, state, handle);
    later call with the same bm, c, s, reverse, chunks and resume_from=handle (plus the now known state_in):
    the per-chunk states computed in step one are reused instead of being computed again.
    resume_swapped=True (dk == dv): the handle comes from the product with bm and c exchanged, whose chunk states are the
    transposes of this one's (dk and dv, forward and dq are such pairs); they are transposed in place and the handle then
    belongs to this product. rebase=False says the kept states already include the incoming state (the handle went through
    a resumed call); state_in must still be passed, in this product's layout, for sequences that are not cut into chunks.
    Any call with keep_workspace=True returns (out, state_out, handle).
    """
    _lib.require_cuda(a, bm, c)
    _lib.raise_on_device_status(bm.device)
    b, h, n, dk = bm.shape
    dv = c.shape[-1]
    dev = bm.device
    bnhd = _use_bnhd(bm, c) if state_only else _use_bnhd(a, bm, c)
    if (resume_from is not None or keep_workspace) and not bnhd and not (bm.is_contiguous() and c.is_contiguous()):
        raise RuntimeError("keep_workspace / resume_from need bm and c in one of the two layouts the library reads in "
                           "place (the handle is tied to their storage)")
    bm = _to_layout(bm, bnhd)
    c = _to_layout(c, bnhd)
    a = None if state_only else _to_layout(a, bnhd)
    sl = _slopes_arg(s, h, dev)
    out = None if state_only else _empty_out(b, h, n, dv, bm.dtype, dev, bnhd)
    dt = _lib.dtype_code(bm.dtype) | (LAYOUT_BNHD if bnhd else 0)
    if state_in is not None:
        state_in = state_in.to(device=dev, dtype=torch.float32).contiguous()
        if tuple(state_in.shape) != (b, h, dv, dk):
            raise RuntimeError(f"state_in must have shape {(b, h, dv, dk)}, got {tuple(state_in.shape)}")
    L = _lib.lib()
    if resume_from is None and (resume_swapped or not rebase):
        raise RuntimeError("resume_swapped / rebase=False need resume_from")
    if resume_from is not None and not resume_swapped and not rebase:
        raise RuntimeError("rebase=False is only available together with resume_swapped")
    if resume_from is not None:
        hd = resume_from
        want_key = _product_key(c, bm, reverse, chunks) if resume_swapped else _product_key(bm, c, reverse, chunks)
        if not isinstance(hd, KeptWorkspace) or hd.key != want_key:
            raise RuntimeError("resume_from does not belong to a call on the same tensors with the same sizes and options")
        if state_in is not None and hd.based == bool(rebase):
            raise RuntimeError("the kept chunk states already include the incoming state" if hd.based else
                               "the kept chunk states do not include the incoming state yet")
        with torch.cuda.device(dev):
            if resume_swapped:
                rc = L.lab200_la_generic_resume_swapped(
                    _lib.ptr(a), _lib.ptr(bm), _lib.ptr(c), _lib.ptr(sl), _lib.ptr(out), _lib.ptr(state_in), hd.ws.data_ptr(),
                    hd.nbytes, b * h, h, n, dk, dv, int(bool(reverse)), int(chunks), int(bool(rebase)),
                    dt, _lib.stream_ptr(dev))
            else:
                rc = L.lab200_la_generic_resume(
                    _lib.ptr(a), _lib.ptr(bm), _lib.ptr(c), _lib.ptr(sl), _lib.ptr(out), _lib.ptr(state_in), hd.ws.data_ptr(),
                    hd.nbytes, b * h, h, n, dk, dv, int(bool(reverse)), int(chunks), dt, _lib.stream_ptr(dev))
        _lib.check(rc, "lab200_la_generic_resume")
        hd.key = _product_key(bm, c, reverse, chunks)  # a swapped resume hands the workspace over to this product
        hd.based = True
        if keep_workspace:
            return out, None, hd
        return out, None
    state_out = torch.empty((b, h, dv, dk), dtype=torch.float32, device=dev) if (want_state or state_only) else None
    with torch.cuda.device(dev):
        nbytes = L.lab200_la_workspace_bytes(b * h, n, dk, dv, chunks)
        ws = _workspace(nbytes, dev)
        rc = L.lab200_la_generic(
            _lib.ptr(a), _lib.ptr(bm), _lib.ptr(c), _lib.ptr(sl), _lib.ptr(out), _lib.ptr(state_in),
            _lib.ptr(state_out), ws.data_ptr(), nbytes, b * h, h, n, dk, dv, int(bool(reverse)),
            int(bool(state_only)), int(chunks), dt, _lib.stream_ptr(dev))
    _lib.check(rc, "lab200_la_generic")
    if keep_workspace:
        return out, state_out, KeptWorkspace(ws, nbytes, _product_key(bm, c, reverse, chunks), based=not state_only)
    return out, state_out


def dkdv_fused_supported(d, e):
    """Shapes the fused dk+dv sweep (lab200_la2_dkdv) covers."""
    return d % 16 == 0 and e % 16 == 0 and 16 <= d <= 128 and 16 <= e <= 128


def la_dkdv(q, k, v, s, do, state_in=None, chunks=0, resume_from=None):
    """dk and dv of the backward pass in one fused reverse-time sweep (lab200_la2_dkdv): q, k, v, do are read once.

    q, k: (b, h, n, d); v, do: (b, h, n, e); d, e <= 128. state_in: optional (b, h, d, e) fp32 reverse-time state
    sum_t lambda^t q_t^T do_t arriving from tokens after the end of the sequence (sequence parallelism).
    resume_from: handle of `la_generic(None, do, q, s, reverse=True, state_only=True, keep_workspace=True, chunks=chunks)`;
    its per-chunk states are reused (the state-only pass over do and q is not repeated). Returns (dk, dv)."""
    _lib.require_cuda(q, k, v, do)
    _lib.raise_on_device_status(q.device)
    b, h, n, d = q.shape
    e = v.shape[-1]
    dev = q.device
    bnhd = _use_bnhd(q, k, v, do)
    if resume_from is not None and not bnhd and not (do.is_contiguous() and q.is_contiguous()):
        raise RuntimeError("resume_from needs do and q in one of the two layouts the library reads in place")
    q, k, v, do = (_to_layout(t, bnhd) for t in (q, k, v, do))
    sl = _slopes_arg(s, h, dev)
    dk = _empty_out(b, h, n, d, q.dtype, dev, bnhd)
    dv = _empty_out(b, h, n, e, q.dtype, dev, bnhd)
    dt = _lib.dtype_code(q.dtype) | (LAYOUT_BNHD if bnhd else 0)
    if state_in is not None:
        state_in = state_in.to(device=dev, dtype=torch.float32).contiguous()
        if tuple(state_in.shape) != (b, h, d, e):
            raise RuntimeError(f"state_in must have shape {(b, h, d, e)}, got {tuple(state_in.shape)}")
    L = _lib.lib()
    with torch.cuda.device(dev):
        if resume_from is not None:
            hd = resume_from
            if not isinstance(hd, KeptWorkspace) or hd.key != _product_key(do, q, True, chunks) or hd.based:
                raise RuntimeError("resume_from does not come from a state-only reverse-time call on (do, q) with the same options")
            ws, nbytes, resume = hd.ws, hd.nbytes, 1
            hd.based = True  # used up: the states now include the incoming state
        else:
            nbytes = L.lab200_la_workspace_bytes(b * h, n, e, d, chunks)
            ws, resume = _workspace(nbytes, dev), 0
        rc = L.lab200_la2_dkdv(q.data_ptr(), k.data_ptr(), v.data_ptr(), _lib.ptr(sl), do.data_ptr(), dk.data_ptr(),
                               dv.data_ptr(), _lib.ptr(state_in), ws.data_ptr(), nbytes, b, h, n, d, e, int(chunks), resume,
                               dt, _lib.stream_ptr(dev))
    _lib.check(rc, "lab200_la2_dkdv")
    return dk, dv


def _fwd(q, k, v, sl, chunks=0, bnhd=False):
    """q, k, v all in one layout: (b, h, n, dim) contiguous, or (bnhd=True) views of (b, n, h, dim) tensors."""
    b, h, n, d = q.shape
    e = v.shape[-1]
    o = _empty_out(b, h, n, e, q.dtype, q.device, bnhd)
    _lib.raise_on_device_status(q.device)
    L = _lib.lib()
    with torch.cuda.device(q.device):
        nbytes = L.lab200_la_workspace_bytes(b * h, n, d, e, chunks)
        ws = _workspace(nbytes, q.device)
        rc = L.lab200_la2_fwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), _lib.ptr(sl), o.data_ptr(), ws.data_ptr(),
                              nbytes, b, h, n, d, e, int(chunks), _lib.dtype_code(q.dtype) | (LAYOUT_BNHD if bnhd else 0),
                              _lib.stream_ptr(q.device))
    _lib.check(rc, "lab200_la2_fwd")
    return o


def _bwd(q, k, v, sl, do, chunks=0, bnhd=False):
    b, h, n, d = q.shape
    e = v.shape[-1]
    dq = _empty_out(b, h, n, d, q.dtype, q.device, bnhd)
    dk = _empty_out(b, h, n, d, q.dtype, q.device, bnhd)
    dv = _empty_out(b, h, n, e, q.dtype, q.device, bnhd)
    _lib.raise_on_device_status(q.device)
    L = _lib.lib()
    with torch.cuda.device(q.device):  # the chunk plan depends on the SM count of the tensors' device
        nbytes = L.lab200_la2_bwd_workspace_bytes(b, h, n, d, e, chunks)
        ws = _workspace(nbytes, q.device)
        rc = L.lab200_la2_bwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), _lib.ptr(sl), do.data_ptr(), dq.data_ptr(),
                              dk.data_ptr(), dv.data_ptr(), ws.data_ptr(), nbytes, b, h, n, d, e, int(chunks),
                              _lib.dtype_code(q.dtype) | (LAYOUT_BNHD if bnhd else 0), _lib.stream_ptr(q.device))
    _lib.check(rc, "lab200_la2_bwd")
    return dq, dk, dv


def _chunked(q, v):
    """True if the library cuts this problem's sequence into chunks (few (batch, head) pairs) and d == e, i.e. when the
    chunk states of one product can be handed to the product with k and v exchanged instead of being recomputed."""
    b, h, n, d = q.shape
    e = v.shape[-1]
    with torch.cuda.device(q.device):
        return d == e and _lib.lib().lab200_la_plan_chunks(b * h, n, d, e) > 1


def _fwd_keep(q, k, v, s):
    """Forward that keeps its chunk states (KV prefixes, (e, d) per chunk) for the backward pass."""
    o, _, handle = la_generic(q, k, v, s, keep_workspace=True)
    return o, handle


def _bwd_from_kept(q, k, v, s, do, handle):
    """Backward in chunk mode with d == e: dq takes the forward's chunk states transposed, dv takes dk's; only dk's
    (reverse-time sums of q^T do) are computed here."""
    dq, _ = la_generic(do, v, k, s, resume_from=handle, resume_swapped=True, rebase=False)
    if dkdv_fused_supported(q.shape[-1], v.shape[-1]):
        return (dq,) + la_dkdv(q, k, v, s, do)
    dk, _, h2 = la_generic(v, do, q, s, reverse=True, keep_workspace=True)
    dv, _ = la_generic(k, q, do, s, reverse=True, resume_from=h2, resume_swapped=True, rebase=False)
    return dq, dk, dv


def _check_inputs(q, k, v):
    _lib.require_cuda(q, k, v)
    if q.dim() != 4 or k.shape != q.shape or v.shape[:3] != q.shape[:3]:
        raise RuntimeError(f"expected q, k (b, h, n, d) and v (b, h, n, e); got {tuple(q.shape)}, {tuple(k.shape)}, {tuple(v.shape)}")
    if not (q.dtype == k.dtype == v.dtype):
        raise RuntimeError("q, k, v must share one dtype")
    if q.dtype not in (torch.bfloat16, torch.float16):
        # the reference's Triton kernels also take fp32 tensors (they compute in fp32 anyway); the tensor-core kernels
        # here read 16-bit operands only, and silently down-casting a caller's fp32 tensors would change its results
        raise RuntimeError(f"lightning attention takes bf16 or fp16 tensors, got {q.dtype}; cast q, k, v first "
                           "(e.g. q.bfloat16()) - accumulation and the running state are fp32 either way")


class LightningAttention2(torch.autograd.Function):
    """o = lightning attention with per-head decay exp(-s) (lightning_attn2.py:398-504)."""

    @staticmethod
    def forward(ctx, q, k, v, s):
        _check_inputs(q, k, v)
        bnhd = _use_bnhd(q, k, v)  # read (b, n, h, dim) projections in place, write o the same way: no transposing copies
        q, k, v = (_to_layout(t, bnhd) for t in (q, k, v))
        s = s.contiguous()
        sl = _slopes_arg(s, q.shape[1], q.device)
        ctx.kept = None
        ctx.bnhd = bnhd
        if _chunked(q, v):
            o, ctx.kept = _fwd_keep(q, k, v, s)
        else:
            o = _fwd(q, k, v, sl, bnhd=bnhd)
        ctx.save_for_backward(q, k, v, s)
        return o

    @staticmethod
    def backward(ctx, do):
        q, k, v, s = ctx.saved_tensors
        do = _to_layout(do, ctx.bnhd)
        kept, ctx.kept = ctx.kept, None  # usable once: the transposed hand-over changes whose states they are
        if kept is not None:
            return _bwd_from_kept(q, k, v, s, do, kept) + (None,)
        sl = _slopes_arg(s, q.shape[1], q.device)
        dq, dk, dv = _bwd(q, k, v, sl, do, bnhd=ctx.bnhd)
        return dq, dk, dv, None


class LightningAttention2NoDecay(torch.autograd.Function):
    """The same without decay (lightning_attn2_no_decay.py:367-468)."""

    @staticmethod
    def forward(ctx, q, k, v):
        _check_inputs(q, k, v)
        bnhd = _use_bnhd(q, k, v)
        q, k, v = (_to_layout(t, bnhd) for t in (q, k, v))
        ctx.kept = None
        ctx.bnhd = bnhd
        if _chunked(q, v):
            o, ctx.kept = _fwd_keep(q, k, v, None)
        else:
            o = _fwd(q, k, v, None, bnhd=bnhd)
        ctx.save_for_backward(q, k, v)
        return o

    @staticmethod
    def backward(ctx, do):
        q, k, v = ctx.saved_tensors
        do = _to_layout(do, ctx.bnhd)
        kept, ctx.kept = ctx.kept, None
        if kept is not None:
            return _bwd_from_kept(q, k, v, None, do, kept)
        dq, dk, dv = _bwd(q, k, v, None, do, bnhd=ctx.bnhd)
        return dq, dk, dv


def lightning_attn_prefill(q, k, v, s=None, kv_state=None):
    """Forward pass that carries the recurrence state, for inference (no autograd; the reference has no such entry).

    q, k: (b, h, n, d); v: (b, h, n, e); d, e multiples of 16, d <= 256; any n. kv_state: None or the (b, h, e, d) fp32
    state entering the first token, i.e. what an earlier call returned. Returns (o, kv_state_out) where kv_state_out
    is the state entering token n: sum_{j<n} lambda^(n-j) k_j^T v_j (transposed) plus the decayed incoming state.
    Feeding it to the next prefill chunk or to `lightning_attn_decode` continues the sequence exactly."""
    _check_inputs(q, k, v)
    with torch.no_grad():
        o, st = la_generic(q.detach(), k.detach(), v.detach(), None if s is None else s.detach(), state_in=kv_state,
                           want_state=True)
    return o, st


def lightning_attn_decode(q, k, v, s, kv_state):
    """One token per (batch, head): o = q (S + k^T v), S <- lambda (S + k^T v), S = kv_state updated IN PLACE.

    q, k: (b, h, d) or (b, h, 1, d); v: (b, h, e) or (b, h, 1, e); kv_state: (b, h, e, d) fp32 contiguous, from
    `lightning_attn_prefill` (or zeros for an empty prefix). Returns o shaped like v. No autograd."""
    _lib.require_cuda(q, k, v, kv_state)
    squeeze = q.dim() == 4
    if squeeze:
        if q.shape[2] != 1 or k.shape[2] != 1 or v.shape[2] != 1:
            raise RuntimeError("lightning_attn_decode takes exactly one token per call")
        q, k, v = q[:, :, 0], k[:, :, 0], v[:, :, 0]
    b, h, d = q.shape
    e = v.shape[-1]
    if k.shape != q.shape or v.shape[:2] != q.shape[:2] or not (q.dtype == k.dtype == v.dtype):
        raise RuntimeError(f"expected q, k (b, h, d) and v (b, h, e) of one dtype; got {tuple(q.shape)}, {tuple(k.shape)}, {tuple(v.shape)}")
    if tuple(kv_state.shape) != (b, h, e, d) or kv_state.dtype != torch.float32 or not kv_state.is_contiguous():
        raise RuntimeError(f"kv_state must be a contiguous fp32 tensor of shape {(b, h, e, d)}")
    q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
    sl = _slopes_arg(s, h, q.device)
    o = torch.empty((b, h, e), dtype=q.dtype, device=q.device)
    with torch.cuda.device(q.device):
        rc = _lib.lib().lab200_la_decode_step(q.data_ptr(), k.data_ptr(), v.data_ptr(), _lib.ptr(sl), kv_state.data_ptr(),
                                              o.data_ptr(), b * h, h, d, e, _lib.dtype_code(q.dtype),
                                              _lib.stream_ptr(q.device))
    _lib.check(rc, "lab200_la_decode_step")
    return o.unsqueeze(2) if squeeze else o


lightning_attn2 = LightningAttention2.apply
lightning_attn2_no_decay = LightningAttention2NoDecay.apply
# The reference's "parallel" variant (lightning_attn2_parallel.py:1072) computes the same function with a
# different kernel decomposition; here the library picks the decomposition itself.
lightning_attn2_parallel = LightningAttention2.apply
