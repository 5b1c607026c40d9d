"""Multi-GPU modes for Lightning Attention-2 (one process per GPU, torch.distributed).

The reference is single-GPU only; both modes below are derived from its recurrences
(lightning_attn/ops/triton/lightning_attn2.py:84 for the forward state, :392-395 for the reverse one).

1. Batch x heads sharding: every (batch, head) pair is an independent scan, so the pairs are split
   contiguously over the ranks and each rank runs the single-GPU op on its share. No communication.

2. Sequence parallelism: the sequence is split into contiguous shards of L tokens (L a multiple of 128),
   one per rank, every rank holding all (batch, head) pairs of its shard. Each rank computes the d x e state
   its shard contributes (from a zero initial state), the states are all-gathered (b*h*d*e fp32 per rank),
   each rank combines the states of the ranks before it with the decay lambda^L per shard,

       KV_in[0] = 0,   KV_in[r] = sum_{j<r} lambda^((r-1-j) L) S_j,

   and runs the single-GPU forward with KV_in[r] as its initial state. The backward pass does the same in
   reverse time for dKV (ranks after r), and reuses KV_in for dq. Per forward+backward that is two all-gathers and two
   one-launch combines; nothing in between waits on the host. The chunk states a product computes on the way are kept
   and reused: by its own block loop once the incoming state is known, and (d == e) by the product with k and v
   exchanged, whose states are the transposes (forward -> dq, dk -> dv).

The device arithmetic is injected as `product` (default: the CUDA op `la_generic`), which keeps the
exchange logic testable on CPU ranks (gloo) with any other implementation of the same product.
"""
import torch
import torch.distributed as dist

BLOCK = 128


# ------------------------------------------------------------------------------------------------
# 1. batch x heads sharding
# ------------------------------------------------------------------------------------------------
def bh_partition(num_units, world_size):
    """Contiguous split of `num_units` (batch, head) pairs: list of (start, stop), sizes differ by at most one."""
    base, rem = divmod(num_units, world_size)
    bounds, start = [], 0
    for r in range(world_size):
        stop = start + base + (1 if r < rem else 0)
        bounds.append((start, stop))
        start = stop
    return bounds


def bh_shard(q, k, v, s, rank, world_size):
    """This rank's share of the (batch, head) pairs of full tensors q, k (b, h, n, d), v (b, h, n, e).

    Returns (q_l, k_l, v_l, s_l) shaped (1, U, n, .) and (U, 1, 1): every local unit becomes its own "head"
    carrying the decay rate of the head it came from, so the single-GPU op applies unchanged."""
    b, h, n, d = q.shape
    start, stop = bh_partition(b * h, world_size)[rank]
    flat = lambda t: t.reshape(b * h, n, t.shape[-1])[start:stop].unsqueeze(0)
    s_l = None
    if s is not None:
        heads = torch.arange(start, stop, device=s.device) % h
        s_l = s.reshape(-1)[:h][heads].reshape(-1, 1, 1)
    return flat(q), flat(k), flat(v), s_l


def lightning_attn_bh_sharded(q, k, v, s=None, group=None):
    """Forward (differentiable) on this rank's share of the (batch, head) pairs; see bh_shard. The result stays
    local, shape (1, U, n, e): no collective is issued."""
    from .ops import lightning_attn_func

    rank = dist.get_rank(group) if dist.is_initialized() else 0
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    q_l, k_l, v_l, s_l = bh_shard(q, k, v, s, rank, world)
    if q_l.shape[1] == 0:
        return q_l.new_zeros((1, 0, q.shape[2], v.shape[-1]))
    return lightning_attn_func(q_l, k_l, v_l, s_l)


# ------------------------------------------------------------------------------------------------
# 2. sequence parallelism
# ------------------------------------------------------------------------------------------------
def _shard_decay(s, h, shard_len, device):
    """lambda^L per head, shape (1, h, 1, 1), fp32 (all ones without decay)."""
    if s is None:
        return torch.ones((1, h, 1, 1), dtype=torch.float32, device=device)
    return torch.exp(-s.detach().to(device=device, dtype=torch.float32).reshape(-1)[:h] * float(shard_len)).reshape(1, h, 1, 1)


def combine_states(states, decay, rank, reverse=False):
    """State entering shard `rank` from the local states of all shards (list indexed by rank, or one stacked tensor).

    forward time: sum_{j<rank} decay^(rank-1-j) states[j];  reverse time: sum_{j>rank} decay^(j-rank-1) states[j].
    Plain torch, any device, no host synchronisation; the CUDA path of `lightning_attn_sp` uses the one-launch kernel
    behind `combine_gathered` instead."""
    stacked = states if torch.is_tensor(states) else torch.stack(list(states), dim=0)  # (R, b, h, x, y)
    R = stacked.shape[0]
    expo = [(j - rank - 1) if reverse else (rank - 1 - j) for j in range(R)]  # >= 0 exactly for the shards that contribute
    if not any(x >= 0 for x in expo):
        return torch.zeros_like(stacked[0])
    h = decay.numel()
    dev = stacked.device
    pw = torch.tensor([max(x, 0) for x in expo], dtype=torch.float32, device=dev).reshape(R, 1)
    use = torch.tensor([x >= 0 for x in expo], device=dev).reshape(R, 1)
    w = decay.reshape(1, h).to(torch.float32) ** pw  # 0 ** 0 == 1
    w = torch.where(use, w, torch.zeros_like(w))
    return torch.einsum("rh,rbhxy->bhxy", w, stacked.to(torch.float32)).to(stacked.dtype)


def gather_states(local_state, group=None):
    """All-gather of the per-rank local states into ONE tensor (world, b, h, x, y): a single collective, no copies."""
    world = dist.get_world_size(group)
    local_state = local_state.contiguous()
    flat = torch.empty((world * local_state.shape[0],) + tuple(local_state.shape[1:]), dtype=local_state.dtype,
                       device=local_state.device)
    dist.all_gather_into_tensor(flat, local_state, group=group)
    return flat.view((world,) + tuple(local_state.shape))


def combine_gathered(gathered, s, shard_len, rank, reverse=False):
    """(state_in, state_in transposed) for shard `rank` from `gather_states` output (world, b, h, x, y).

    CUDA tensors: one launch of the library's combine kernel (lab200_la_combine_states) writes both layouts.
    Other devices (the gloo tests of the exchange logic): the torch formula of `combine_states`."""
    R, b, h, x, y = gathered.shape
    if gathered.is_cuda:
        from . import _lib

        dev = gathered.device
        g = gathered.to(torch.float32).contiguous()
        sl = None if s is None else s.detach().to(device=dev, dtype=torch.float32).reshape(-1)[:h].contiguous()
        out = torch.empty((b, h, x, y), dtype=torch.float32, device=dev)
        out_t = torch.empty((b, h, y, x), dtype=torch.float32, device=dev)
        with torch.cuda.device(dev):
            rc = _lib.lib().lab200_la_combine_states(g.data_ptr(), _lib.ptr(sl), out.data_ptr(), out_t.data_ptr(), R, rank,
                                                     b * h, h, x, y, int(shard_len), int(bool(reverse)), _lib.stream_ptr(dev))
        _lib.check(rc, "lab200_la_combine_states")
        return out, out_t
    out = combine_states(gathered, _shard_decay(s, h, shard_len, gathered.device), rank, reverse=reverse)
    return out, out.transpose(2, 3).contiguous()


def _default_product():
    from .ops.cuda.lightning_attn2 import la_generic

    return la_generic


class _SequenceParallelAttention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, s, group, product, dkdv):
        b, h, L, d = q.shape
        if L % BLOCK != 0:
            raise RuntimeError(f"sequence-parallel shards must be multiples of {BLOCK} tokens, got {L}")
        rank = dist.get_rank(group)
        # state this shard contributes, (b, h, e, d) = KV^T, from a zero initial state; the per-chunk states computed
        # on the way are kept and reused by the second call, which then only runs the block loop
        _, s_loc, handle = product(None, k, v, s, reverse=False, state_only=True, keep_workspace=True)
        kv_in, kv_in_t = combine_gathered(gather_states(s_loc, group), s, L, rank, reverse=False)
        o, _, handle = product(q, k, v, s, reverse=False, state_in=kv_in, resume_from=handle, keep_workspace=True)
        ctx.save_for_backward(q, k, v, s if s is not None else torch.empty(0), kv_in_t)
        ctx.has_s = s is not None
        ctx.group, ctx.product, ctx.dkdv = group, product, dkdv
        ctx.kv_handle = handle if d == v.shape[-1] else None  # chunk states of (k, v), incoming state included
        return o

    @staticmethod
    def backward(ctx, do):
        q, k, v, s, kv_in_t = ctx.saved_tensors
        s = s if ctx.has_s else None
        group, product = ctx.group, ctx.product
        b, h, L, d = q.shape
        rank = dist.get_rank(group)
        do = do.contiguous()
        # dq_t = sum_{j<=t} lambda^(t-j) (do_t . v_j) k_j : forward time, incoming state = KV_in in (d, e) layout. Its chunk
        # states are the transposes of the forward's, which are still in the kept workspace (used once: a second backward
        # through the same graph recomputes them).
        handle, ctx.kv_handle = ctx.kv_handle, None
        if handle is not None:
            dq, _ = product(do, v, k, s, reverse=False, state_in=kv_in_t, resume_from=handle, resume_swapped=True, rebase=False)
        else:
            dq, _ = product(do, v, k, s, reverse=False, state_in=kv_in_t)
        # reverse-time state of this shard for dk: (b, h, d, e) = sum_t lambda^t q_t^T do_t
        _, ds_loc, handle = product(None, do, q, s, reverse=True, state_only=True, keep_workspace=True)
        dkv_in, dkv_in_t = combine_gathered(gather_states(ds_loc, group), s, L, rank, reverse=True)
        if ctx.dkdv is not None:  # one fused sweep for dk and dv; the kept chunk states of (do, q) are rebased on dkv_in
            dk, dv = ctx.dkdv(q, k, v, s, do, state_in=dkv_in, resume_from=handle)
            return dq, dk, dv, None, None, None, None
        dk, _, handle = product(v, do, q, s, reverse=True, state_in=dkv_in, resume_from=handle, keep_workspace=True)
        if d == v.shape[-1]:
            dv, _ = product(k, q, do, s, reverse=True, state_in=dkv_in_t, resume_from=handle, resume_swapped=True, rebase=False)
        else:
            dv, _ = product(k, q, do, s, reverse=True, state_in=dkv_in_t)
        return dq, dk, dv, None, None, None, None


def lightning_attn_sp(q, k, v, s=None, group=None, product=None, dkdv=None):
    """Sequence-parallel lightning attention. q, k (b, h, L, d) and v (b, h, L, e) are this rank's contiguous
    shard of the sequence (rank r holds tokens [r L, (r+1) L)); returns this rank's shard of o. Differentiable
    w.r.t. q, k, v; two all-gathers of (b, h, d, e) fp32 states per forward+backward.
    `product` / `dkdv`: implementations of the generic product and of the fused dk+dv sweep (signatures of `la_generic` and
    `la_dkdv`); default: the CUDA ops, with the fused sweep wherever it covers the shape."""
    if not dist.is_initialized():
        raise RuntimeError("lightning_attn_sp needs an initialised torch.distributed process group")
    if product is None:
        product = _default_product()
        from .ops.cuda.lightning_attn2 import dkdv_fused_supported, la_dkdv

        if dkdv is None and dkdv_fused_supported(q.shape[-1], v.shape[-1]):
            dkdv = la_dkdv
    return _SequenceParallelAttention.apply(q.contiguous(), k.contiguous(), v.contiguous(), s, group, product, dkdv)
