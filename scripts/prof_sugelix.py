"""ncu target: one launch each (after one warm-up each) of the rotary step over segments and of the fixed-layout kernel
at the same shape, and of the capped 16-bit prefill attention and the uncapped one.
usage: python scripts/prof_sugelix.py [tokens]"""
import sys

import torch

sys.path.insert(0, ".")
from semi_pd_b200 import ops  # noqa: E402
from semi_pd_b200.rimidra import _rotary_table  # noqa: E402

dev, bf = torch.device("cuda:0"), torch.bfloat16
T = int(sys.argv[1]) if len(sys.argv) > 1 else 16384
H, G, D, L = 16, 4, 128, 2048
torch.manual_seed(0)
sizes = [H * D, G * D, G * D]
wide = torch.randn(T, sum(sizes) + H * D, device=dev, dtype=bf)
q, k, v = wide[:, : sum(sizes)].split(sizes, -1)
qb, kb, vb = (torch.randn(n, device=dev) for n in sizes)
slots = T + 8
kp, vp = torch.zeros(slots, G * D, device=dev, dtype=bf), torch.zeros(slots, G * D, device=dev, dtype=bf)
q_out = torch.empty(T, H * D, device=dev, dtype=bf)
table = _rotary_table(D, 1e6, L + 64, dev)
locs = torch.arange(1, T + 1, device=dev)
pos = torch.arange(T, device=dev) % L
segs = [ops.rotary_segment(q, q_out, H, D, D, bias=qb), ops.rotary_segment(k, kp, G, D, D, bias=kb, to_pool=True),
        ops.rotary_segment(v, vp, G, D, 0, bias=vb, to_pool=True)]
n_req = 4
r2t = (torch.arange(n_req * L, device=dev, dtype=torch.int32) + 1).view(n_req, L).contiguous()
rpi = torch.arange(n_req, device=dev)
pre = torch.zeros(n_req, dtype=torch.int32, device=dev)
ext = torch.full((n_req,), L, dtype=torch.int32, device=dev)
start = torch.arange(n_req, device=dev, dtype=torch.int32) * L
qa = torch.randn(n_req * L, H * D, device=dev, dtype=bf)
kpa, vpa = torch.randn(slots, G, D, device=dev, dtype=bf), torch.randn(slots, G, D, device=dev, dtype=bf)


def attention(cap):
    ops.attn_general(qa, kpa, vpa, r2t, rpi, H, G, D, D, D ** -0.5, prefix_lens=pre, extend_lens=ext,
                     extend_start_loc=start, max_extend_len=L, softcap=cap)


for _ in range(2):  # the first pass over the four kernels warms up
    ops.rotary_segments(segs, pos, table, bf, loc=locs, paired=True)
    ops.rotary_bias_store(q, k, v, qb, kb, kp.view(slots, G, D), vp.view(slots, G, D), locs, pos, table, D, H, G, D, D)
    attention(30.0)
    attention(0.0)
torch.cuda.synchronize()
