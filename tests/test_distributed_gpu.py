"""Multi-GPU test (needs >= 2 GPUs, skipped otherwise): sequence-parallel forward+backward over NCCL with the
CUDA kernels against the single-GPU result. Ranks leave only after all work is done; NVLS is switched off."""
import os
import socket
import sys

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, scale, result_dir):
    import torch.distributed as dist

    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        import lightning_attention_b200 as la
        from lightning_attention_b200 import distributed as D

        torch.manual_seed(5)
        b, h, L, d, e = 1, 8, 512, 128, 128
        n = world * L
        mk = lambda *shape: (0.5 * torch.randn(*shape)).to(torch.bfloat16).to(dev)
        q, k, v, do = mk(b, h, n, d), mk(b, h, n, d), mk(b, h, n, e), mk(b, h, n, e)
        s = None if scale == 0 else (la._build_slope_tensor(h) * scale).to(dev)
        sl = slice(rank * L, (rank + 1) * L)
        ql, kl, vl = (t[:, :, sl].contiguous().requires_grad_() for t in (q, k, v))
        o = D.lightning_attn_sp(ql, kl, vl, s)
        o.backward(do[:, :, sl].contiguous())
        qf, kf, vf = (t.clone().requires_grad_() for t in (q, k, v))
        of = la.lightning_attn_func(qf, kf, vf, s)
        of.backward(do)
        torch.cuda.synchronize()

        def rel(x, y):
            x, y = x.float(), y.float()
            return float((x - y).norm() / (y.norm() + 1e-30))

        errs = [rel(o, of[:, :, sl]), rel(ql.grad, qf.grad[:, :, sl]), rel(kl.grad, kf.grad[:, :, sl]),
                rel(vl.grad, vf.grad[:, :, sl])]
        np.save(os.path.join(result_dir, f"err_{rank}.npy"), np.asarray(errs))
        dist.barrier()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("scale", [1.0, 1e-3, 0.0])
def test_sequence_parallel_nccl(tmp_path, scale):
    world = min(torch.cuda.device_count(), 4)
    if world < 2:
        pytest.skip("needs at least 2 GPUs")
    import torch.multiprocessing as mp

    mp.spawn(_worker, args=(world, _free_port(), scale, str(tmp_path)), nprocs=world, join=True)
    for r in range(world):
        errs = np.load(tmp_path / f"err_{r}.npy")
        # both sides are bf16 CUDA results of the same math with different chunk boundaries
        assert np.all(errs < 1e-2), (r, errs)
