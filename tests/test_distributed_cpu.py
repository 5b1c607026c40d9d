"""CPU tests (gloo, world_size 2 and 4) of the multi-GPU host logic: the batch x heads partition and the
sequence-parallel state exchange. The device product is replaced by the numpy oracle so no GPU is needed;
the exchange, the decayed combination and the autograd wiring are the code under test."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def oracle_product(a, bm, c, s=None, reverse=False, state_in=None, want_state=False, state_only=False, chunks=0,
                   keep_workspace=False, resume_from=None, resume_swapped=False, rebase=True):
    """Same call signature as the CUDA op `la_generic`, computed by the numpy oracle in fp64. The two-step protocol
    (keep_workspace / resume_from / resume_swapped) is honoured by handing back a token that names the product it belongs
    to and whether the incoming state is already in it, and checking the token that comes back."""
    from oracle import lightning_oracle as O

    f = lambda t: None if t is None else t.detach().double().numpy()
    a_ = f(a) if a is not None else np.zeros_like(f(bm))
    out, st = O.la_generic(a_, f(bm), f(c), f(s), reverse=reverse, state_in=f(state_in))
    out_t = None if state_only else torch.from_numpy(np.ascontiguousarray(out))
    st_t = torch.from_numpy(np.ascontiguousarray(st)).float().double()
    if resume_from is not None:
        tag, bshape, cshape, rev, based = resume_from
        want = (tuple(c.shape), tuple(bm.shape)) if resume_swapped else (tuple(bm.shape), tuple(c.shape))
        assert (tag, bshape, cshape, rev) == ("handle",) + want + (bool(reverse),)
        assert based == (not rebase), "the incoming state must be added exactly once"
    if keep_workspace:
        based = (state_in is not None) or (resume_from is not None)
        return out_t, st_t, ("handle", tuple(bm.shape), tuple(c.shape), bool(reverse), based)
    return out_t, st_t


def oracle_dkdv(q, k, v, s, do, state_in=None, chunks=0, resume_from=None):
    """Same call signature as the CUDA op `la_dkdv` (fused dk + dv sweep), computed by the numpy oracle as the two
    reverse-time products it fuses; state_in is the (b, h, d, e) reverse-time state, and a handle must come from a
    state-only reverse-time call on (do, q) that has not had an incoming state added yet."""
    from oracle import lightning_oracle as O

    f = lambda t: None if t is None else t.detach().double().numpy()
    if resume_from is not None:
        tag, bshape, cshape, rev, based = resume_from
        assert (tag, bshape, cshape, rev, based) == ("handle", tuple(do.shape), tuple(q.shape), True, False)
    st = f(state_in)
    dk, _ = O.la_generic(f(v), f(do), f(q), f(s), reverse=True, state_in=st)
    dv, _ = O.la_generic(f(k), f(q), f(do), f(s), reverse=True, state_in=None if st is None else np.swapaxes(st, -1, -2))
    return torch.from_numpy(np.ascontiguousarray(dk)), torch.from_numpy(np.ascontiguousarray(dv))


def _sp_worker(rank, world, port, scale, result_dir, d=16, e=32, fused=False):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from lightning_attention_b200 import distributed as D
        from oracle import lightning_oracle as O

        torch.manual_seed(11)
        b, h, L = 1, 3, 128
        n = world * L
        q, k = (torch.randn(b, h, n, d, dtype=torch.float64) for _ in range(2))
        v, do = (torch.randn(b, h, n, e, dtype=torch.float64) for _ in range(2))
        s = None if scale == 0 else torch.from_numpy(O.build_slopes(h)).double().reshape(h, 1, 1) * scale
        sl = slice(rank * L, (rank + 1) * L)
        ql, kl, vl = (t[:, :, sl].clone().requires_grad_() for t in (q, k, v))
        o = D.lightning_attn_sp(ql, kl, vl, s, product=oracle_product, dkdv=oracle_dkdv if fused else None)
        o.backward(do[:, :, sl])
        sn = None if s is None else s.numpy()
        ro = O.linear_attn(q.numpy(), k.numpy(), v.numpy(), sn)
        rdq, rdk, rdv = O.linear_attn_bwd(q.numpy(), k.numpy(), v.numpy(), sn, do.numpy())
        errs = [O.max_abs_err(o.detach().numpy(), ro[:, :, sl]), O.max_abs_err(ql.grad.numpy(), rdq[:, :, sl]),
                O.max_abs_err(kl.grad.numpy(), rdk[:, :, sl]), O.max_abs_err(vl.grad.numpy(), rdv[:, :, sl])]
        np.save(os.path.join(result_dir, f"err_{rank}.npy"), np.asarray(errs))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
@pytest.mark.parametrize("scale", [1.0, 1e-3, 0.0])
def test_sequence_parallel_matches_unsharded(tmp_path, world, scale):
    """Each rank's output and gradients equal its slice of the unsharded result (decay 1x, 1e-3x so that the
    incoming state matters everywhere, and none)."""
    mp.spawn(_sp_worker, args=(world, _free_port(), scale, str(tmp_path)), nprocs=world, join=True)
    for r in range(world):
        errs = np.load(tmp_path / f"err_{r}.npy")
        # the oracle product hands back fp32-rounded states (as the CUDA op does); 1e-4 absolute covers that
        assert np.all(errs < 1e-4), (r, errs)


def test_sequence_parallel_square_dims_reuse_transposed_states(tmp_path):
    """d == e: dq resumes from the forward's kept chunk states and dv from dk's, both through the transposed hand-over;
    the product stand-in checks every handle it is given (right product, incoming state added exactly once)."""
    world = 2
    mp.spawn(_sp_worker, args=(world, _free_port(), 1e-3, str(tmp_path), 32, 32), nprocs=world, join=True)
    for r in range(world):
        errs = np.load(tmp_path / f"err_{r}.npy")
        assert np.all(errs < 1e-4), (r, errs)


@pytest.mark.parametrize("scale", [1e-3, 0.0])
def test_sequence_parallel_with_the_fused_dk_dv_sweep(tmp_path, scale):
    """The backward branch the CUDA path takes for d, e <= 128: one state-only pass over (do, q), the exchange, then ONE
    fused call for dk and dv that takes the combined incoming state and the kept handle."""
    world = 2
    mp.spawn(_sp_worker, args=(world, _free_port(), scale, str(tmp_path), 16, 32, True), nprocs=world, join=True)
    for r in range(world):
        errs = np.load(tmp_path / f"err_{r}.npy")
        assert np.all(errs < 1e-4), (r, errs)


def _fail_worker(rank, world, port, result_dir):
    """Rank 1 raises before the exchange; rank 0's all-gather must end with an error (short timeout), not hang."""
    import datetime

    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=5))
    from lightning_attention_b200 import distributed as D

    outcome = "completed"
    try:
        if rank == 1:
            raise ValueError("injected host-side failure before the state exchange")
        D.gather_states(torch.zeros(1, 2, 4, 4))
    except ValueError:
        outcome = "raised"
    except Exception:
        outcome = "exchange_error"
    with open(os.path.join(result_dir, f"outcome_{rank}.txt"), "w") as f:
        f.write(outcome)
    try:
        dist.destroy_process_group()
    except Exception:
        pass


def test_exchange_fails_cleanly_when_a_rank_drops_out(tmp_path):
    mp.spawn(_fail_worker, args=(2, _free_port(), str(tmp_path)), nprocs=2, join=True)
    assert (tmp_path / "outcome_1.txt").read_text() == "raised"
    assert (tmp_path / "outcome_0.txt").read_text() == "exchange_error"


def test_bh_partition_and_shard():
    sys.path.insert(0, ROOT)
    from lightning_attention_b200 import distributed as D

    assert D.bh_partition(128, 8) == [(16 * r, 16 * (r + 1)) for r in range(8)]
    parts = D.bh_partition(10, 4)
    assert parts == [(0, 3), (3, 6), (6, 8), (8, 10)]
    b, h, n, d = 2, 3, 5, 4
    q = torch.arange(b * h * n * d, dtype=torch.float32).reshape(b, h, n, d)
    s = torch.tensor([0.5, 0.25, 0.125]).reshape(h, 1, 1)
    seen = []
    for r in range(4):
        ql, kl, vl, sl = D.bh_shard(q, q, q, s, r, 4)
        start, stop = D.bh_partition(b * h, 4)[r]
        assert ql.shape == (1, stop - start, n, d)
        assert torch.equal(ql[0], q.reshape(b * h, n, d)[start:stop])
        assert torch.equal(sl.reshape(-1), s.reshape(-1)[torch.arange(start, stop) % h])
        seen += list(range(start, stop))
    assert seen == list(range(b * h))


def test_combine_states_formula():
    sys.path.insert(0, ROOT)
    from lightning_attention_b200 import distributed as D

    states = [torch.full((1, 2, 1, 1), float(i + 1)) for i in range(4)]
    decay = torch.tensor([0.5, 1.0]).reshape(1, 2, 1, 1)
    # forward, rank 3: 0.25*S0 + 0.5*S1 + S2 for head 0; S0+S1+S2 for head 1
    got = D.combine_states(states, decay, 3)
    assert torch.allclose(got.reshape(-1), torch.tensor([0.25 * 1 + 0.5 * 2 + 3, 6.0]))
    assert float(D.combine_states(states, decay, 0).abs().sum()) == 0.0
    # reverse, rank 0: S1 + 0.5*S2 + 0.25*S3
    got = D.combine_states(states, decay, 0, reverse=True)
    assert torch.allclose(got.reshape(-1), torch.tensor([2 + 0.5 * 3 + 0.25 * 4, 9.0]))
    assert float(D.combine_states(states, decay, 3, reverse=True).abs().sum()) == 0.0
