"""Flex attention under the planner: a block with a sliding-window causal mask and grouped-query heads on a
2-D mesh.  The planner may replicate the attention call, split its batch or split its heads per mesh dim; the
block mask (built with ``B=None, H=None``) stays replicated.  Prints the placements chosen for the two
higher-order operators and runs one local forward / backward of rank 0's graph.
(Reference counterpart: tests/test_flex_attention.py of the reference, which covers the same operators.)"""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import torch
import torch.nn as nn
from torch.distributed.tensor.placement_types import Replicate, Shard
from torch.nn.attention.flex_attention import create_block_mask, flex_attention

from autoparallel_b200 import AutoParallel
from autoparallel_b200.parallel.strategies.flex_rules import is_flex_attention_node
from examples._fake import fake_mesh

WINDOW = 256


def sliding_window_causal(b, h, q, kv):
    return (q >= kv) & (q - kv < WINDOW)


class Block(nn.Module):
    def __init__(self, d=512, heads=8, kv_heads=4):
        super().__init__()
        self.h, self.kvh, self.hd = heads, kv_heads, d // heads
        self.norm = nn.LayerNorm(d)
        self.wq = nn.Linear(d, d, bias=False)
        self.wkv = nn.Linear(d, 2 * kv_heads * self.hd, bias=False)
        self.wo = nn.Linear(d, d, bias=False)

    def forward(self, x):
        B, S, _ = x.shape
        y = self.norm(x)
        q = self.wq(y).view(B, S, self.h, self.hd).transpose(1, 2)
        k, v = self.wkv(y).view(B, S, 2, self.kvh, self.hd).permute(2, 0, 3, 1, 4)
        mask = create_block_mask(sliding_window_causal, None, None, S, S, device=x.device)
        o = flex_attention(q, k, v, block_mask=mask, enable_gqa=True)
        return x + self.wo(o.transpose(1, 2).reshape(B, S, -1))


def main():
    mesh = fake_mesh((2, 4), ("dp", "tp"))
    with torch.device("meta"):
        model = Block()
    with AutoParallel(model, lambda: torch.randn(8, 1024, 512), mesh) as ap:
        ap.add_parameter_memory_constraint()
        ap.add_input_constraints([(Shard(0), Replicate())])
        ap.add_output_constraints([(Shard(0), Replicate())])
        sol = ap.optimize_placement()
        for n in ap.joint.gm.graph.nodes:
            if is_flex_attention_node(n):
                spec = sol[n]
                print(f"{n.target.name():26s} q {tuple(spec.input_specs[0].placements)}  k {tuple(spec.input_specs[1].placements)}"
                      f"  out {tuple(spec.output_specs[0].placements)}")
        parallel = ap.apply_placement()
    parallel.to_empty(device="cpu")
    with torch.no_grad():
        for p in parallel.parameters():
            p._local_tensor.normal_(std=0.02)
    y = parallel(torch.randn(4, 1024, 512))
    y.sum().backward()
    print("local output", tuple(y.shape), "gradients:", sum(p.grad is not None for p in parallel.parameters()), "of", len(list(parallel.parameters())))


if __name__ == "__main__":
    main()
