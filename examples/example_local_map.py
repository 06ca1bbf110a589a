"""Manual parallelism inside an automatically planned model: context-parallel attention as a
``local_map`` region on a 3-D (dp, tp, cp) mesh, with an all-gather of K/V over the ``cp`` axis so
the region computes full (non-causal) attention for its query shard.
(Reference counterpart: examples/example_local_map.py – whose region does local attention only.)"""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import torch
import torch.nn as nn
import torch.nn.functional as F
from torch.distributed.tensor.placement_types import Replicate, Shard

from autoparallel_b200 import AutoParallel
from autoparallel_b200.collectives import all_gather, local_map
from examples._fake import fake_mesh


def cp_attention(k, v, q):  # local [B/dp, H/tp, S/cp, D]; arguments in order of first use (capture requires it)
    k = all_gather(k, "cp", gather_dim=2)
    v = all_gather(v, "cp", gather_dim=2)
    return F.scaled_dot_product_attention(q, k, v, is_causal=False)


class Attn(nn.Module):
    def __init__(self, d=512, heads=8):
        super().__init__()
        self.heads = heads
        self.qkv = nn.Linear(d, 3 * d, bias=False)
        self.o = nn.Linear(d, d, bias=False)

    def forward(self, x):
        b, s, d = x.shape
        q, k, v = (t.view(b, s, self.heads, -1).transpose(1, 2) for t in self.qkv(x).chunk(3, -1))
        pl = (Shard(0), Shard(1), Shard(2))
        a = local_map(cp_attention, out_placements=(pl,), in_placements=(pl, pl, pl))(k, v, q)
        return self.o(a.transpose(1, 2).reshape(b, s, d))


def main():
    mesh = fake_mesh((2, 2, 2), ("dp", "tp", "cp"))
    with torch.device("meta"):
        model = Attn()
    with AutoParallel(model, lambda: torch.randn(8, 256, 512), mesh) as autop:
        autop.add_input_constraints([(Shard(0), Replicate(), Shard(1))])
        autop.optimize_placement()
        lowered = autop.lower()
        print("collectives:", lowered.num_collectives)


if __name__ == "__main__":
    main()
