"""fp8 projections under the planner: a two-layer MLP whose linears quantise activations and weights row-wise to
float8_e4m3fn and multiply them with ``torch._scaled_mm``.  On 8 fake ranks (2 x 4 mesh) the pattern pass rewrites the
calls to ``apb200::scaled_mm`` and the solver shards the rows of the activations together with their row-wise scales
(the quantised weights are small buffers here and stay replicated; pinned to a column split with ``add_node_constraint``
their scales would follow them, and the fusion pass would merge a gathered fp8 operand with its scale, or the
reduce-scatter of a row-parallel product, into one node - ``tests/test_fp8_scaled_mm.py`` exercises those forms).

    python examples/example_fp8_linear.py

(Reference counterpart: the fp8 patterns of autoparallel/graph_passes/async_tp/asynctp.py:390-537 and the scaled fused
operators of asynctp_ops.py:948-1026, 1189-1424.)"""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import torch
import torch.nn as nn
from torch.distributed.tensor.placement_types import Replicate, Shard

from autoparallel_b200 import AutoParallel
from examples._fake import fake_mesh

F8 = torch.float8_e4m3fn


def quant_rows(t):
    scale = t.abs().amax(dim=-1, keepdim=True).clamp(min=1e-6) / 448.0
    return (t / scale).to(F8), scale


class Fp8Linear(nn.Module):
    """Inference-style fp8 linear: the weight is quantised once (buffers), the activation on the fly."""

    def __init__(self, d_in, d_out):
        super().__init__()
        self.register_buffer("wq", torch.zeros(d_out, d_in).to(F8))
        self.register_buffer("sw", torch.ones(d_out, 1))

    def forward(self, x):
        with torch.no_grad():
            xq, sx = quant_rows(x)
        return torch._scaled_mm(xq, self.wq.t(), scale_a=sx, scale_b=self.sw.t(), out_dtype=torch.bfloat16)


class Model(nn.Module):
    def __init__(self, d=1024, h=4096):
        super().__init__()
        self.up, self.down = Fp8Linear(d, h), Fp8Linear(h, d)
        self.head = nn.Linear(d, d, bias=False, dtype=torch.bfloat16)      # a trainable layer behind the frozen fp8 ones

    def forward(self, x):
        return self.head(self.down(torch.nn.functional.gelu(self.up(x)))).float().square().mean()


def main():
    mesh = fake_mesh((2, 4), ("dp", "tp"))
    with torch.device("meta"):
        model = Model()
    with AutoParallel(model, lambda: torch.randn(8192, 1024, dtype=torch.bfloat16), mesh, fuse_collectives=True) as ap:
        print("pattern pass:", {k: v for k, v in ap.joint.pattern_stats.items() if v})
        ap.add_parameter_memory_constraint()
        ap.add_input_constraints([(Shard(0), Replicate())])
        ap.optimize_placement()
        low = ap.lower()
        print("collectives:", dict(low.num_collectives), "fused:", {k: v for k, v in ap.fusion_stats.items() if v})
        apb = torch.ops.apb200
        for n in ap.joint.gm.graph.nodes:
            if n.op == "call_function" and n.target is apb.scaled_mm.default:
                spec = ap.sharding_optimizer.solution[n] if hasattr(ap.sharding_optimizer, "solution") else None
                if spec is not None:
                    ins = [tuple(s.placements) for s in spec.input_specs]
                    print(f"{n.name}: out {tuple(spec.output_specs.placements)}  a {ins[0]}  b {ins[1]}  scale_a {ins[2]}  scale_b {ins[3]}")


if __name__ == "__main__":
    main()
