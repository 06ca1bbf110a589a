"""Smallest end-to-end use of the API: a transformer-ish block on a fake 8 x 8 mesh.
(Reference counterpart: examples/example_autoparallel.py.)

    python examples/example_autoparallel.py
"""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import torch
import torch.nn as nn
from torch.distributed.tensor.placement_types import Replicate, Shard

from autoparallel_b200 import AutoParallel
from examples._fake import fake_mesh


class Block(nn.Module):
    def __init__(self, d=1024, heads=16):
        super().__init__()
        self.heads = heads
        self.wq, self.wk, self.wv, self.wo = (nn.Linear(d, d, bias=False) for _ in range(4))
        self.w1, self.w2 = nn.Linear(d, 4 * d), nn.Linear(4 * d, d)

    def forward(self, x):
        b, s, d = x.shape
        q, k, v = (w(x).view(b, s, self.heads, -1).transpose(1, 2) for w in (self.wq, self.wk, self.wv))
        a = torch.nn.functional.scaled_dot_product_attention(q, k, v, is_causal=True).transpose(1, 2).reshape(b, s, d)
        x = x + self.wo(a)
        return x + self.w2(torch.relu(self.w1(x)))

    def init_weights(self):
        for m in self.modules():
            if isinstance(m, nn.Linear):
                nn.init.normal_(m.weight, std=0.02)
                if m.bias is not None:
                    nn.init.zeros_(m.bias)


def main():
    mesh = fake_mesh((8, 8), ("dp", "tp"))
    with torch.device("meta"):
        model = Block()
    with AutoParallel(model, lambda: torch.randn(512, 256, 1024), mesh, plan_device="B200") as autop:
        autop.add_parameter_memory_constraint()
        autop.add_input_constraints([(Shard(0), Replicate())])
        autop.add_output_constraints([(Shard(0), Replicate())])
        placement = autop.optimize_placement()
        print(autop.sharding_optimizer.get_log()[-400:])
        parallel = autop.apply_placement(placement)
        print("collectives in the per-rank graph:", autop.lowered.num_collectives, "fused:", autop.fusion_stats)
    parallel.to_empty(device="cpu")
    parallel.init_weights()
    out = parallel(torch.randn(512 // 8, 256, 1024))  # local shard of the batch
    out.sum().backward()
    print("ran one local step; output shard", tuple(out.shape), "isinstance(parallel, Block):", isinstance(parallel, Block))


if __name__ == "__main__":
    main()
