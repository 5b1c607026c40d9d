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
   reverse time for dKV (ranks after r), and reuses KV_in for dq.

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
    """State entering shard `rank` from the local states of all shards (list indexed by rank).

    forward time: sum_{j<rank} decay^(rank-1-j) states[j];  reverse time: sum_{j>rank} decay^(j-rank-1) states[j].
    One stacked weighted sum (a handful of kernel launches whatever the number of ranks)."""
    R = len(states)
    idx = torch.arange(R, device=states[0].device)
    expo = (idx - rank - 1) if reverse else (rank - 1 - idx)  # >= 0 exactly for the shards that contribute
    use = expo >= 0
    if not bool(use.any()):
        return torch.zeros_like(states[0])
    h = decay.numel()
    w = decay.reshape(1, h).to(torch.float32) ** expo.clamp(min=0).reshape(R, 1).to(torch.float32)  # 0 ** 0 == 1
    w = torch.where(use.reshape(R, 1), w, torch.zeros_like(w))
    stacked = torch.stack([t.to(torch.float32) for t in states], dim=0)  # (R, b, h, x, y)
    return torch.einsum("rh,rbhxy->bhxy", w, stacked).to(states[0].dtype)


def exchange_states(local_state, group=None):
    """All-gather of the per-rank local states (each (b, h, x, y) fp32). Returns the list indexed by rank."""
    world = dist.get_world_size(group)
    out = [torch.empty_like(local_state) for _ in range(world)]
    dist.all_gather(out, local_state.contiguous(), group=group)
    return out


def _default_product():
    from .ops.cuda.lightning_attn2 import la_generic

    return la_generic


class _SequenceParallelAttention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, s, group, product):
        b, h, L, d = q.shape
        if L % BLOCK != 0:
            raise RuntimeError(f"sequence-parallel shards must be multiples of {BLOCK} tokens, got {L}")
        rank = dist.get_rank(group)
        decay = _shard_decay(s, h, L, q.device)
        # state this shard contributes, (b, h, e, d) = KV^T, from a zero initial state; the per-chunk states computed
        # on the way are kept and reused by the second call, which then only runs the block loop
        _, s_loc, handle = product(None, k, v, s, reverse=False, state_only=True, keep_workspace=True)
        kv_in = combine_states(exchange_states(s_loc, group), decay, rank, reverse=False)
        o, _ = product(q, k, v, s, reverse=False, state_in=kv_in, resume_from=handle)
        ctx.save_for_backward(q, k, v, s if s is not None else torch.empty(0), kv_in)
        ctx.has_s = s is not None
        ctx.group, ctx.product = group, product
        return o

    @staticmethod
    def backward(ctx, do):
        q, k, v, s, kv_in = ctx.saved_tensors
        s = s if ctx.has_s else None
        group, product = ctx.group, ctx.product
        b, h, L, d = q.shape
        rank = dist.get_rank(group)
        decay = _shard_decay(s, h, L, q.device)
        do = do.contiguous()
        # dq_t = sum_{j<=t} lambda^(t-j) (do_t . v_j) k_j : forward time, incoming state = KV_in (d x e layout)
        dq, _ = product(do, v, k, s, reverse=False, state_in=kv_in.transpose(2, 3).contiguous())
        # reverse-time state of this shard for dk: (b, h, d, e) = sum_t lambda^t q_t^T do_t
        _, ds_loc, handle = product(None, do, q, s, reverse=True, state_only=True, keep_workspace=True)
        dkv_in = combine_states(exchange_states(ds_loc, group), decay, rank, reverse=True)
        dk, _ = product(v, do, q, s, reverse=True, state_in=dkv_in, resume_from=handle)
        dv, _ = product(k, q, do, s, reverse=True, state_in=dkv_in.transpose(2, 3).contiguous())
        return dq, dk, dv, None, None, None


def lightning_attn_sp(q, k, v, s=None, group=None, product=None):
    """Sequence-parallel lightning attention. q, k (b, h, L, d) and v (b, h, L, e) are this rank's contiguous
    shard of the sequence (rank r holds tokens [r L, (r+1) L)); returns this rank's shard of o. Differentiable
    w.r.t. q, k, v; two all-gathers of (b, h, d, e) fp32 states per forward+backward."""
    if not dist.is_initialized():
        raise RuntimeError("lightning_attn_sp needs an initialised torch.distributed process group")
    if product is None:
        product = _default_product()
    return _SequenceParallelAttention.apply(q.contiguous(), k.contiguous(), v.contiguous(), s, group, product)
