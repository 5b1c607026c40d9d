"""A TransNormer-style attention block on top of the B200 ops, showing the two caller-side fusions.

Same structure as the reference's example block (examples/module/tnl_attn.py:12-74: q/k/v projections, SiLU,
lightning attention with per-layer-scaled slopes, normalisation, sigmoid output gate, output projection), with two
differences in how the attention op is fed and drained:

* the projections are viewed as (b, h, n, d) without copying; the op reads that (b, n, h, d) memory in place and
  writes its output the same way, so `out.transpose(1, 2).reshape(b, n, h * d)` is free;
* normalisation and gate are one fused kernel, `srmsnorm_sigmoid_gate` (SimpleRMSNorm, the normalisation this
  library provides, stands where the reference's example uses nn.LayerNorm).

`fused=False` runs the same arithmetic the unfused way (contiguous copies, separate norm, sigmoid and multiply), which
is what the tests compare against.
"""
import torch
import torch.nn as nn
import torch.nn.functional as F

import lightning_attention_b200 as la


class TnlAttentionB200(nn.Module):
    def __init__(self, embed_dim, num_heads, bias=False, layer_idx=0, num_layers=12, fused=True):
        super().__init__()
        if embed_dim % num_heads:
            raise ValueError("embed_dim must be a multiple of num_heads")
        self.num_heads = num_heads
        self.head_dim = embed_dim // num_heads
        self.fused = fused
        self.q_proj = nn.Linear(embed_dim, embed_dim, bias=bias)
        self.k_proj = nn.Linear(embed_dim, embed_dim, bias=bias)
        self.v_proj = nn.Linear(embed_dim, embed_dim, bias=bias)
        self.gate_down = nn.Linear(embed_dim, self.head_dim, bias=bias)
        self.gate_up = nn.Linear(self.head_dim, embed_dim, bias=bias)
        self.o_proj = nn.Linear(embed_dim, embed_dim, bias=bias)
        self.norm = la.SimpleRMSNorm(embed_dim)
        # later layers decay more slowly (tnl_attn.py:36-38)
        slopes = la._build_slope_tensor(num_heads) * (1 - layer_idx / (num_layers - 1) + 1e-5)
        self.register_buffer("slope_rate", slopes, persistent=False)

    def forward(self, x):
        b, n, _ = x.shape
        h, d = self.num_heads, self.head_dim
        q, k, v = (F.silu(proj(x)).view(b, n, h, d) for proj in (self.q_proj, self.k_proj, self.v_proj))
        gate = self.gate_up(self.gate_down(x))
        if self.fused:
            # (b, n, h, d) tensors viewed as (b, h, n, d): read and written in place by the op, no copy anywhere
            q, k, v = (t.transpose(1, 2) for t in (q, k, v))
            o = la.lightning_attn_func(q, k, v, self.slope_rate)
            o = o.transpose(1, 2).reshape(b, n, h * d)  # no copy: o is laid out (b, n, h, d)
            y = la.srmsnorm_sigmoid_gate(o, gate, self.norm.eps)
        else:
            q, k, v = (t.transpose(1, 2).contiguous() for t in (q, k, v))
            o = la.lightning_attn_func(q, k, v, self.slope_rate)
            o = o.transpose(1, 2).reshape(b, n, h * d)  # a transposing copy
            y = self.norm(o) * torch.sigmoid(gate)
        return self.o_proj(y)
