"""The example attention block (examples/tnl_attention.py): fused feeding/draining of the op against the unfused way."""
import os
import sys

import pytest
import torch

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "examples"))

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("embed,heads,n", [(1024, 8, 1024), (768, 12, 300)])
def test_fused_block_matches_unfused_block(cuda_lib, embed, heads, n):
    from tnl_attention import TnlAttentionB200

    torch.manual_seed(5)
    blk = TnlAttentionB200(embed, heads, layer_idx=3).cuda().bfloat16()
    x = (torch.randn(2, n, embed, device="cuda") * 0.5).bfloat16().requires_grad_()
    dy = torch.randn(2, n, embed, device="cuda").bfloat16()
    outs = {}
    for fused in (True, False):
        blk.fused = fused
        blk.zero_grad(set_to_none=True)
        x.grad = None
        y = blk(x)
        y.backward(dy)
        outs[fused] = (y.detach().float(), x.grad.float(), blk.q_proj.weight.grad.float(), blk.gate_up.weight.grad.float())
    for a, r, name in zip(outs[True], outs[False], ("y", "dx", "dW_q", "dW_gate")):
        rel = float((a - r).norm() / (r.norm() + 1e-20))
        assert rel < 2e-2, (name, rel)
